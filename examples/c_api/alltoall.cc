// AlltoAll: block j of rank i's send buffer becomes block i of rank j's receive buffer.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 5000;                            // elements per (source, destination) pair
        std::vector<int32_t> in(count * c.size), out(count * c.size);
        for (uint32_t j = 0; j < c.size; ++j)
            for (uint64_t i = 0; i < count; ++i) in[j * count + i] = (int32_t)(c.rank * 100 + j);
        void *din = c.Alloc(in.size() * 4), *dout = c.Alloc(out.size() * 4);
        c.Upload(din, in.data(), in.size() * 4);
        HCCLCHECK(HcclAlltoAll(din, count, HCCL_DATA_TYPE_INT32, dout, count, HCCL_DATA_TYPE_INT32, c.comm, c.stream));
        c.Sync();
        c.Download(out.data(), dout, out.size() * 4);
        c.Free(din);
        c.Free(dout);
        for (uint32_t s = 0; s < c.size; ++s)
            for (uint64_t i = 0; i < count; ++i) if (out[s * count + i] != (int32_t)(s * 100 + c.rank)) return false;
        return true;
    });
}
