// AllGather: rank r contributes a block filled with r; every rank receives the blocks in rank order.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 65537;
        std::vector<uint16_t> mine(count, (uint16_t)c.rank), all(count * c.size);
        void *in = c.Alloc(count * 2), *out = c.Alloc(count * 2 * c.size);
        c.Upload(in, mine.data(), count * 2);
        HCCLCHECK(HcclAllGather(in, out, count, HCCL_DATA_TYPE_UINT16, c.comm, c.stream));
        c.Sync();
        c.Download(all.data(), out, count * 2 * c.size);
        c.Free(in);
        c.Free(out);
        for (uint32_t r = 0; r < c.size; ++r)
            for (uint64_t i = 0; i < count; ++i) if (all[r * count + i] != r) return false;
        return true;
    });
}
