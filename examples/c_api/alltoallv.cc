// AlltoAllV: rank i sends (i + j + 1) * 100 elements to rank j; counts and displacements are per-rank arrays.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        auto cnt = [](uint32_t from, uint32_t to) { return (uint64_t)(from + to + 1) * 100; };
        std::vector<uint64_t> sc(c.size), sd(c.size), rc(c.size), rd(c.size);
        uint64_t so = 0, ro = 0;
        for (uint32_t j = 0; j < c.size; ++j) {
            sc[j] = cnt(c.rank, j); sd[j] = so; so += sc[j];
            rc[j] = cnt(j, c.rank); rd[j] = ro; ro += rc[j];
        }
        std::vector<int64_t> in(so), out(ro);
        for (uint32_t j = 0; j < c.size; ++j)
            for (uint64_t i = 0; i < sc[j]; ++i) in[sd[j] + i] = (int64_t)c.rank * 1000000 + j * 1000 + (int64_t)(i % 1000);
        void *din = c.Alloc(so * 8), *dout = c.Alloc(ro * 8);
        c.Upload(din, in.data(), so * 8);
        HCCLCHECK(HcclAlltoAllV(din, sc.data(), sd.data(), HCCL_DATA_TYPE_INT64, dout, rc.data(), rd.data(), HCCL_DATA_TYPE_INT64, c.comm, c.stream));
        c.Sync();
        c.Download(out.data(), dout, ro * 8);
        c.Free(din);
        c.Free(dout);
        for (uint32_t s = 0; s < c.size; ++s)
            for (uint64_t i = 0; i < rc[s]; ++i)
                if (out[rd[s] + i] != (int64_t)s * 1000000 + c.rank * 1000 + (int64_t)(i % 1000)) return false;
        return true;
    });
}
