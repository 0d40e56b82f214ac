// Scatter from the last rank: block r of the root's send buffer goes to rank r.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 77777;
        const uint32_t root = c.size - 1;
        std::vector<float> in, out(count);
        void *din = nullptr;
        if (c.rank == root) {
            in.resize(count * c.size);
            for (uint32_t b = 0; b < c.size; ++b)
                for (uint64_t i = 0; i < count; ++i) in[b * count + i] = (float)b + 0.5f;
            din = c.Alloc(in.size() * 4);
            c.Upload(din, in.data(), in.size() * 4);
        }
        void *dout = c.Alloc(count * 4);
        HCCLCHECK(HcclScatter(din, dout, count, HCCL_DATA_TYPE_FP32, root, c.comm, c.stream));
        c.Sync();
        c.Download(out.data(), dout, count * 4);
        if (din) c.Free(din);
        c.Free(dout);
        for (float v : out) if (v != (float)c.rank + 0.5f) return false;
        return true;
    });
}
