// Broadcast from rank 1: every rank ends up with the root's buffer.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 300001;
        const uint32_t root = c.size > 1 ? 1 : 0;
        std::vector<int32_t> host(count);
        for (uint64_t i = 0; i < count; ++i) host[i] = (int32_t)(c.rank * 1000 + i % 997);
        void *buf = c.Alloc(count * 4);
        c.Upload(buf, host.data(), count * 4);
        HCCLCHECK(HcclBroadcast(buf, count, HCCL_DATA_TYPE_INT32, root, c.comm, c.stream));
        c.Sync();
        c.Download(host.data(), buf, count * 4);
        c.Free(buf);
        for (uint64_t i = 0; i < count; ++i) if (host[i] != (int32_t)(root * 1000 + i % 997)) return false;
        return true;
    });
}
