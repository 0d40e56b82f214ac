// Ring exchange with HcclBatchSendRecv: every rank sends to rank+1 and receives from rank-1 in ONE call, the building
// block of pipeline parallelism and of ring attention.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 100000;
        std::vector<int32_t> host(count, (int32_t)c.rank);
        void *sendBuf = c.Alloc(count * 4), *recvBuf = c.Alloc(count * 4);
        c.Upload(sendBuf, host.data(), count * 4);
        HcclSendRecvItem items[2] = {
            {HCCL_SEND, sendBuf, count, HCCL_DATA_TYPE_INT32, (c.rank + 1) % c.size},
            {HCCL_RECV, recvBuf, count, HCCL_DATA_TYPE_INT32, (c.rank + c.size - 1) % c.size},
        };
        HCCLCHECK(HcclBatchSendRecv(items, 2, c.comm, c.stream));
        c.Sync();
        c.Download(host.data(), recvBuf, count * 4);
        c.Free(sendBuf);
        c.Free(recvBuf);
        for (int32_t v : host) if (v != (int32_t)((c.rank + c.size - 1) % c.size)) return false;
        return true;
    });
}
