// AllReduce(sum) of 1 Mi floats: every rank contributes rank+1, every element becomes size*(size+1)/2.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 1 << 20;
        std::vector<float> host(count, (float)(c.rank + 1));
        void *in = c.Alloc(count * 4), *out = c.Alloc(count * 4);
        c.Upload(in, host.data(), count * 4);
        HCCLCHECK(HcclAllReduce(in, out, count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, c.comm, c.stream));
        c.Sync();
        c.Download(host.data(), out, count * 4);
        c.Free(in);
        c.Free(out);
        const float want = (float)(c.size * (c.size + 1) / 2);
        for (float v : host) if (v != want) return false;
        return true;
    });
}
