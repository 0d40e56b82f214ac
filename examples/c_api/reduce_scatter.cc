// ReduceScatter(sum): the input holds one block per rank; rank r receives the sum of everybody's block r.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 40000;                           // elements per block
        std::vector<float> in(count * c.size), out(count);
        for (uint32_t b = 0; b < c.size; ++b)
            for (uint64_t i = 0; i < count; ++i) in[b * count + i] = (float)(b + 1) * (float)(c.rank + 1);
        void *din = c.Alloc(in.size() * 4), *dout = c.Alloc(count * 4);
        c.Upload(din, in.data(), in.size() * 4);
        HCCLCHECK(HcclReduceScatter(din, dout, count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, c.comm, c.stream));
        c.Sync();
        c.Download(out.data(), dout, count * 4);
        c.Free(din);
        c.Free(dout);
        const float want = (float)(c.rank + 1) * (float)(c.size * (c.size + 1) / 2);
        for (float v : out) if (v != want) return false;
        return true;
    });
}
