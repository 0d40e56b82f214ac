// Point to point: even ranks send 1 MiB of floats to rank+1, odd ranks receive from rank-1.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 256 * 1024;
        if (c.size % 2 && c.rank == c.size - 1) return true;     // odd world: the last rank has no partner
        std::vector<float> host(count, (float)c.rank);
        void *buf = c.Alloc(count * sizeof(float));
        c.Upload(buf, host.data(), count * sizeof(float));
        if (c.rank % 2 == 0) HCCLCHECK(HcclSend(buf, count, HCCL_DATA_TYPE_FP32, c.rank + 1, c.comm, c.stream));
        else HCCLCHECK(HcclRecv(buf, count, HCCL_DATA_TYPE_FP32, c.rank - 1, c.comm, c.stream));
        c.Sync();
        c.Download(host.data(), buf, count * sizeof(float));
        c.Free(buf);
        float want = (float)(c.rank % 2 == 0 ? c.rank : c.rank - 1);
        for (float v : host) if (v != want) return false;
        return true;
    });
}
