// AlltoAllVC: the same exchange described by ONE count matrix that every rank passes (matrix[i][j] = elements i -> j);
// buffers are packed in rank order, so no displacement arrays are needed.
#include "common.h"

int main()
{
    return RunRanks([](RankCtx &c) {
        std::vector<uint64_t> M(c.size * c.size);
        for (uint32_t i = 0; i < c.size; ++i)
            for (uint32_t j = 0; j < c.size; ++j) M[i * c.size + j] = (uint64_t)((i * 3 + j * 5) % 4) * 250;   // zeros included
        uint64_t so = 0, ro = 0;
        for (uint32_t j = 0; j < c.size; ++j) { so += M[c.rank * c.size + j]; ro += M[j * c.size + c.rank]; }
        std::vector<float> in(so + 1), out(ro + 1, -1.f);
        uint64_t o = 0;
        for (uint32_t j = 0; j < c.size; ++j)
            for (uint64_t i = 0; i < M[c.rank * c.size + j]; ++i) in[o++] = (float)(c.rank * 64 + j);
        void *din = c.Alloc((so + 1) * 4), *dout = c.Alloc((ro + 1) * 4);
        c.Upload(din, in.data(), (so + 1) * 4);
        HCCLCHECK(HcclAlltoAllVC(din, M.data(), HCCL_DATA_TYPE_FP32, dout, HCCL_DATA_TYPE_FP32, c.comm, c.stream));
        c.Sync();
        c.Download(out.data(), dout, (ro + 1) * 4);
        c.Free(din);
        c.Free(dout);
        o = 0;
        for (uint32_t s = 0; s < c.size; ++s)
            for (uint64_t i = 0; i < M[s * c.size + c.rank]; ++i) if (out[o++] != (float)(s * 64 + c.rank)) return false;
        return true;
    });
}
