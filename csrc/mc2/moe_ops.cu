// Host side of the MoE dispatch / combine operators: symmetric workspace layout, launches, emulation entry.
#include "../common/launch_count.h"
#include <cuda_fp8.h>
#include <algorithm>
#include "../common/log.h"
#include "../core/comm.h"
#include "../kernels/emu_world.h"
#include "hccl/hccl_moe.h"
#include "moe_kernels.cuh"

namespace hccl {
namespace moe {

namespace {

uint64_t Al(uint64_t v) { return (v + 255) & ~255ull; }

HcclResult CheckConfig(const HcclMoeConfig &c, uint32_t nranks)
{
    if (c.numExperts == 0 || c.numExperts > (uint32_t)kMaxExperts || c.numExperts % nranks) { HCCL_ERROR("MoE: numExperts %u must be a multiple of the rank count and at most %d", c.numExperts, kMaxExperts); return HCCL_E_PARA; }
    if (c.topK == 0 || c.topK > 16) { HCCL_ERROR("MoE: topK %u outside [1, 16]", c.topK); return HCCL_E_PARA; }
    if (c.hidden == 0 || c.hidden % 256) { HCCL_ERROR("MoE: hidden %u must be a multiple of 256", c.hidden); return HCCL_E_PARA; }
    if (c.maxTokens == 0 || c.maxTokens >= (1u << 24)) { HCCL_ERROR("MoE: maxTokens %u outside [1, 2^24)", c.maxTokens); return HCCL_E_PARA; }
    return HCCL_SUCCESS;
}

uint32_t Capacity(const HcclMoeConfig &c) { return c.maxRecvRows ? c.maxRecvRows : 2 * c.maxTokens * c.topK; }

MoeLayout MakeLayout(const HcclMoeConfig &c, uint32_t maxCtas)
{
    MoeLayout L{};
    const uint64_t cap = Capacity(c), entries = (uint64_t)c.maxTokens * c.topK;
    uint64_t off = 0;
    L.recvX = off; off += Al(cap * c.hidden * (c.mxfp8 ? 1 : 2));
    L.recvScales = off; off += Al(c.mxfp8 ? cap * (c.hidden / 32) : 0);
    L.recvSrc = off; off += Al(cap * 4);
    L.yBuf = off; off += Al(cap * c.hidden * 2);
    L.recvCounts = off; off += Al((uint64_t)kMaxExperts * 4);
    L.pos = off; off += Al(entries * 4);
    L.slotMap = off; off += Al(entries * 8);
    L.cntCta = off; off += Al((uint64_t)maxCtas * c.numExperts * 4);
    L.baseSend = off; off += Al((uint64_t)kMaxExperts * 4);
    L.total = off;
    return L;
}

struct MoeState {
    Comm *comm = nullptr;
    HcclMoeConfig cfg{};
    MoeLayout L{};
    void *ws = nullptr;
    uint64_t wsOff = 0;
    uint32_t ctas = 0;
    uint32_t lastTokens = 0;
};

int SmCountNow()
{
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

MoeArgs MakeArgs(const HcclMoeConfig &cfg, const MoeLayout &L, uint64_t wsOff, uint32_t T)
{
    MoeArgs a{};
    a.T = T; a.K = cfg.topK; a.H = cfg.hidden; a.E = cfg.numExperts; a.cap = Capacity(cfg); a.mxfp8 = cfg.mxfp8;
    a.wsOff = wsOff;
    a.L = L;
    return a;
}

template <bool EMU> HcclResult LaunchMoe(bool dispatch, const DevComm *comms, const MoeArgs &a, const MoeArgs *emuArgs, uint32_t ctas, uint32_t ranksY, cudaStream_t s)
{
    const void *fn = dispatch ? (const void *)MoeDispatchKernel<EMU> : (const void *)MoeCombineKernel<EMU>;
    MoeArgs av = a;
    void *params[] = {(void *)&comms, (void *)&av, (void *)&emuArgs};
    cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(ctas, ranksY), dim3(kMoeThreads), params, 0, s);
    if (e != cudaSuccess) { HCCL_ERROR("MoE kernel launch failed: %s (grid %u x %u)", cudaGetErrorString(e), ctas, ranksY); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

}  // namespace
}  // namespace moe
}  // namespace hccl

using namespace hccl;
using namespace hccl::moe;

extern "C" {

HcclResult HcclMoeCreate(HcclComm comm, const HcclMoeConfig *config, HcclMoeHandle *handle)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !config || !handle) return HCCL_E_PTR;
    if (c->backend != BackendKind::CUDA) { HCCL_ERROR("MoE dispatch / combine need a CUDA communicator"); return HCCL_E_NOT_SUPPORT; }
    CHK_RET(CheckConfig(*config, c->nranks));
    auto *st = new MoeState();
    st->comm = c;
    st->cfg = *config;
    // leave SMs for the expert GEMMs of the neighbouring streams; all CTAs must be co-resident (cooperative launch)
    st->ctas = (uint32_t)std::min(SmCountNow(), 64);
    if (const char *e = getenv("HCCL_MOE_CTAS")) { int v = atoi(e); if (v > 0 && v <= SmCountNow()) st->ctas = (uint32_t)v; }
    st->L = MakeLayout(*config, st->ctas);
    HcclResult r = SymAlloc(c, st->L.total, &st->ws);
    if (r != HCCL_SUCCESS) { delete st; return r; }
    st->wsOff = SymOffsetOf(c, st->ws);
    *handle = st;
    return c->boot->Barrier();
}

HcclResult HcclMoeDestroy(HcclMoeHandle handle)
{
    auto *st = (MoeState *)handle;
    if (!st) return HCCL_E_PTR;
    cudaDeviceSynchronize();
    if (CommFromHandle(st->comm)) SymFree(st->comm, st->ws);
    delete st;
    return HCCL_SUCCESS;
}

HcclResult HcclMoeDispatch(HcclMoeHandle handle, const void *x, const int32_t *topkIdx, uint32_t numTokens, void **recvX, void **recvScales,
                           int32_t **recvCounts, int32_t **recvSrc, cudaStream_t stream)
{
    auto *st = (MoeState *)handle;
    if (!st || !x || !topkIdx) return HCCL_E_PTR;
    if (numTokens == 0 || numTokens > st->cfg.maxTokens) { HCCL_ERROR("MoE dispatch: %u tokens, configured maximum %u", numTokens, st->cfg.maxTokens); return HCCL_E_PARA; }
    Comm *c = st->comm;
    CHK_RET(CommCheckReady(c));
    MoeArgs a = MakeArgs(st->cfg, st->L, st->wsOff, numTokens);
    a.x = x;
    a.topkIdx = topkIdx;
    CHK_RET(LaunchMoe<false>(true, c->devCommPtr, a, nullptr, st->ctas, 1, stream));
    st->lastTokens = numTokens;
    c->counters.kernelsLaunched++;
    CountLaunch();
    c->counters.ops++;
    char *ws = (char *)st->ws;
    if (recvX) *recvX = ws + st->L.recvX;
    if (recvScales) *recvScales = st->cfg.mxfp8 ? ws + st->L.recvScales : nullptr;
    if (recvCounts) *recvCounts = (int32_t *)(ws + st->L.recvCounts);
    if (recvSrc) *recvSrc = (int32_t *)(ws + st->L.recvSrc);
    return HCCL_SUCCESS;
}

HcclResult HcclMoeGetExpertOutBuffer(HcclMoeHandle handle, void **y)
{
    auto *st = (MoeState *)handle;
    if (!st || !y) return HCCL_E_PTR;
    *y = (char *)st->ws + st->L.yBuf;
    return HCCL_SUCCESS;
}

HcclResult HcclMoeCombine(HcclMoeHandle handle, const float *topkWeights, void *out, uint32_t numTokens, cudaStream_t stream)
{
    auto *st = (MoeState *)handle;
    if (!st || !topkWeights || !out) return HCCL_E_PTR;
    if (numTokens != st->lastTokens) { HCCL_ERROR("MoE combine: %u tokens but the last dispatch routed %u", numTokens, st->lastTokens); return HCCL_E_PARA; }
    Comm *c = st->comm;
    CHK_RET(CommCheckReady(c));
    MoeArgs a = MakeArgs(st->cfg, st->L, st->wsOff, numTokens);
    a.weights = topkWeights;
    a.out = out;
    CHK_RET(LaunchMoe<false>(false, c->devCommPtr, a, nullptr, st->ctas, 1, stream));
    c->counters.kernelsLaunched++;
    CountLaunch();
    c->counters.ops++;
    return HCCL_SUCCESS;
}

HcclResult HcclEmuMoeRoundTrip(void *emu, const HcclMoeConfig *config, void **xs, void **idxs, void **weights, void **outs, uint32_t numTokens,
                               void **recvCountsOut, uint32_t ctasPerRank)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !config || !xs || !idxs || !weights || !outs) return HCCL_E_PTR;
    uint32_t R = (uint32_t)w->nranks;
    CHK_RET(CheckConfig(*config, R));
    MoeLayout L = MakeLayout(*config, ctasPerRank);
    if (L.total > w->arenaBytes) { HCCL_ERROR("emu arena too small for MoE: need %llu bytes", (unsigned long long)L.total); return HCCL_E_MEMORY; }
    if (sizeof(MoeArgs) * R > 2048 * R) return HCCL_E_INTERNAL;
    std::vector<MoeArgs> args(R);
    for (int pass = 0; pass < 2; ++pass) {
        for (uint32_t r = 0; r < R; ++r) {
            args[r] = MakeArgs(*config, L, w->arenaOff, numTokens);
            args[r].x = xs[r];
            args[r].topkIdx = (const int32_t *)idxs[r];
            args[r].weights = (const float *)weights[r];
            args[r].out = outs[r];
            args[r].identity = 1;
        }
        if (cudaMemcpy(w->devFusedParams, args.data(), sizeof(MoeArgs) * R, cudaMemcpyHostToDevice) != cudaSuccess) return HCCL_E_RUNTIME;
        CHK_RET(LaunchMoe<true>(pass == 0, w->devComms, args[0], (const MoeArgs *)w->devFusedParams, ctasPerRank, R, 0));
        if (cudaStreamSynchronize(0) != cudaSuccess) { HCCL_ERROR("emu MoE kernel failed: %s", cudaGetErrorString(cudaGetLastError())); return HCCL_E_RUNTIME; }
        for (uint32_t r = 0; r < R; ++r) if (w->status[r].code != 0) return w->status[r].code == 2 ? HCCL_E_MEMORY : HCCL_E_TIMEOUT;
    }
    if (recvCountsOut)
        for (uint32_t r = 0; r < R; ++r)
            if (recvCountsOut[r]) cudaMemcpy(recvCountsOut[r], w->heaps[r] + w->arenaOff + L.recvCounts, (config->numExperts / R) * 4, cudaMemcpyDeviceToDevice);
    return HCCL_SUCCESS;
}

}  // extern "C"
