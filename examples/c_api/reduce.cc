// Reduce(max) to rank 0: only the root's output buffer is written.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 12345;
        std::vector<int32_t> in(count), out(count, -7);
        for (uint64_t i = 0; i < count; ++i) in[i] = (int32_t)((i * 31 + c.rank * 17) % 1000);
        void *din = c.Alloc(count * 4), *dout = c.Alloc(count * 4);
        c.Upload(din, in.data(), count * 4);
        c.Upload(dout, out.data(), count * 4);
        HCCLCHECK(HcclReduce(din, dout, count, HCCL_DATA_TYPE_INT32, HCCL_REDUCE_MAX, 0, c.comm, c.stream));
        c.Sync();
        c.Download(out.data(), dout, count * 4);
        c.Free(din);
        c.Free(dout);
        for (uint64_t i = 0; i < count; ++i) {
            int32_t want = -7;
            if (c.rank == 0) {
                want = 0;
                for (uint32_t r = 0; r < c.size; ++r) want = std::max(want, (int32_t)((i * 31 + r * 17) % 1000));
            }
            if (out[i] != want) return false;
        }
        return true;
    });
}
