// AllReduce on registered memory: HcclMemAlloc hands out a block of the communicator's symmetric heap that is already a
// registered window (the same offset on every rank when all ranks allocate in the same order), so from 1 MB up the
// operator lets the switch / the peers address the buffer directly instead of staging through the scratch buffer.
// Every rank contributes rank + 1 in 4 Mi floats, reduces in place, and checks size * (size + 1) / 2.
// (On the simulation backend the block is host memory and the operator stages as always; the calls are the same.)
#include "common.h"
#include "hccl/hccl_res.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 4u << 20;
        void *buf = nullptr;
        HCCLCHECK(HcclMemAlloc(c.comm, count * 4, &buf));
        std::vector<float> host(count, (float)(c.rank + 1));
        c.Upload(buf, host.data(), count * 4);
        HCCLCHECK(HcclAllReduce(buf, buf, count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, c.comm, c.stream));
        c.Sync();
        c.Download(host.data(), buf, count * 4);
        // a range inside the block is a window too; outside the heap it is refused
        uint64_t off = 0;
        HCCLCHECK(HcclCommMemReg(c.comm, (char *)buf + 4096, 8192, &off));
        float onStack[4];
        if (HcclCommMemReg(c.comm, onStack, sizeof(onStack), &off) != HCCL_E_NOT_SUPPORT) return false;
        HCCLCHECK(HcclMemFree(c.comm, buf));
        const float want = (float)(c.size * (c.size + 1) / 2);
        for (float v : host) if (v != want) return false;
        return true;
    });
}
