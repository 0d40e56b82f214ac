// Host side of the fused matmul + collective operators: argument checks, symmetric workspace, tensor maps, launch.
// Real communicators launch one kernel per rank (cooperatively, so every CTA of the op is resident); the emulation
// entry launches one kernel for all ranks of a single-GPU world.
#include "../common/launch_count.h"
#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>
#include "../common/dtype.h"
#include "../common/log.h"
#include "../core/comm.h"
#include "../exec/op_common.h"
#include "../kernels/emu_world.h"
#include "fused_policies.cuh"
#include "gemm_sm100_2cta.cuh"
#include "gemm_sm100_mx.cuh"
#include "gemm_sm100_mx_2cta.cuh"
#include "gemm_host.h"
#include "hccl/hccl_mc2.h"

namespace hccl {
namespace mc2 {

namespace {

enum FusedKind { AGMM = 0, MMRS = 1, MMAR = 2 };

struct FusedShape {
    FusedKind kind;
    uint32_t n, rank;
    uint64_t m, N, K;          // AGMM: m = mLocal; MMRS/MMAR: m = full M, K = kLocal
    bool mx = false;           // block-scaled fp8 operands (e4m3 + e8m0 scale atoms) instead of bf16
};

// bytes of the scale atoms that go with `rows` x K block-scaled elements (rows a multiple of 128)
uint64_t SfBytes(uint64_t rows, uint64_t K) { return ((rows + 127) / 128) * (K / 128) * 512; }

// workspace bytes per parity half
uint64_t WorkspaceHalfBytes(const FusedShape &s)
{
    switch (s.kind) {
        case AGMM: return s.mx ? (uint64_t)s.n * s.m * s.K + SfBytes((uint64_t)s.n * s.m, s.K) : (uint64_t)s.n * s.m * s.K * 2;
        case MMRS: return (uint64_t)s.m * s.N * 2;                       // n slots of (m/n) x N
        default: return (uint64_t)s.n * s.m * (s.N / s.n) * 2 + (uint64_t)s.m * s.N * 2;   // partial slots + result window
    }
}

uint32_t CommCtasDefault()
{
    if (const char *e = getenv("HCCL_MC2_COMM_CTAS")) { int v = atoi(e); if (v > 0 && v < 64) return (uint32_t)v; }
    return 8;
}

template <int BN, class Policy, bool EMU> HcclResult SetSmemAttrMx()
{
    static std::atomic<bool> done{false};
    if (!done) {
        auto kern = GemmKernelMx<BN, Policy, EMU>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmMxSmem<BN>::kTotal + 1024) != cudaSuccess) return HCCL_E_RUNTIME;
        done = true;
    }
    return HCCL_SUCCESS;
}

template <int BN, class Policy, bool EMU> HcclResult SetSmemAttr()
{
    static std::atomic<bool> done{false};
    if (!done) {
        auto kern = GemmKernel<BN, Policy, EMU>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::kTotal + 1024) != cudaSuccess) return HCCL_E_RUNTIME;
        done = true;
    }
    return HCCL_SUCCESS;
}

// Fills everything except the DevComm pointer. heapLocal = this rank's heap base as mapped here.
// The CTA-pair (cta_group::2) kernel serves AllGatherMatmul and MatmulReduceScatter when every rank's rows split into
// whole 256-row pairs. HCCL_MC2_CTA_PAIR=0 keeps the one-CTA kernels.
// HCCL_MC2_CTA_PAIR: 0 = one-CTA kernels only; 1 = AllGatherMatmul and MatmulReduceScatter on CTA pairs with 256-wide
// tiles (AllGatherMatmul keeps its communication CTAs); 2 = also 224-wide tiles where they waste fewer waves;
// 3 = AllGatherMatmul without communication CTAs, warps 2 and 3 of every GEMM CTA push the shard (measured slower at 2 GPUs:
// the pushes of all CTAs contend with the operand loads during the first hundred microseconds).
// Unset: pairs on 2 ranks (measured +1..3 % on the 2-GPU step), one-CTA kernels on more ranks (at 8 GPUs the per-rank
// GEMMs are short and the pair kernels measured 0..3 % slower: 1.019-1.029 ms against 0.997-1.016 ms per step).
int PairLevel(uint32_t nranks = 2)
{
    static const int level = [] { const char *e = getenv("HCCL_MC2_CTA_PAIR"); return e ? atoi(e) : -1; }();
    if (level >= 0) return level;
    return nranks <= 2 ? 1 : 0;
}

// Block-scaled operators: CTA pairs by default (HCCL_MX_PAIR=0 keeps the one-CTA kernel); MatmulAllReduce stays one-CTA.
bool MxPairEnabled()
{
    const char *e = getenv("HCCL_MX_PAIR");
    return !(e && e[0] == '0');
}

bool PairModeFor(const FusedShape &s)
{
    if (s.mx) {
        if (!MxPairEnabled() || s.N < 256 || s.kind == MMAR) return false;
        return s.kind == AGMM ? (s.m / kBM) % 2 == 0 : (s.m / s.n / kBM) % 2 == 0;
    }
    if (PairLevel(s.n) <= 0 || s.N < 256) return false;
    if (s.kind == AGMM) return (s.m / kBM) % 2 == 0;
    if (s.kind == MMRS) return (s.m / s.n / kBM) % 2 == 0;
    return false;
}

// Tile width of the CTA-pair kernels: 256, or 224 when that needs less work-in-waves on `pairs` CTA pairs.
uint32_t PairTileN(uint64_t rowPairs, uint64_t N, uint32_t pairs)
{
    auto cost = [&](uint32_t bn) { uint64_t tiles = rowPairs * ((N + bn - 1) / bn); return ((tiles + pairs - 1) / pairs) * bn; };
    return PairLevel() >= 2 && cost(224) < cost(256) ? 224u : 256u;
}

// Tile width of the block-scaled AllGatherMatmul / MatmulReduceScatter: 256 (one accumulator in tensor memory) or 192 (two, the
// epilogue overlaps the next main loop). HCCL_MX_TILE_N overrides; read on every call so that tests can switch it.
uint32_t MxTileN()
{
    const char *e = getenv("HCCL_MX_TILE_N");
    const int v = e ? atoi(e) : 0;
    return v == 192 ? 192u : v == 256 ? 256u : kMxDefaultTileN;
}

// Block-scaled form: a / b are e4m3 payloads, sfa / sfb their scale atoms; MxTileN()-wide tiles (128-wide for MatmulAllReduce).
HcclResult BuildParamsMx(const FusedShape &s, char *heapLocal, uint64_t wsOff, const void *a, const void *sfa, const void *b, const void *sfb, void *out,
                         uint32_t commCtas, GemmParams *p, uint32_t pairBN = 0)
{
    memset(p, 0, sizeof(*p));
    const uint64_t half = WorkspaceHalfBytes(s);
    const uint32_t bn = pairBN ? pairBN : MxTileN();       // tile width; a CTA of a pair loads half of the B tile
    const uint32_t boxB = pairBN ? pairBN / 2 : bn;
    const uint64_t kAtoms = s.K / 128;
    p->errorWord = GemmErrorWord();
    p->groupM = 16;
    p->elemBytes = 1;
    p->sfA = (const uint8_t *)sfa;
    p->sfB = (const uint8_t *)sfb;
    p->sfAtomsB = (uint32_t)((s.N + 127) / 128);
    p->N = (uint32_t)s.N; p->K = (uint32_t)s.K; p->ldc = (uint32_t)s.N; p->C = out;
    if (s.kind == AGMM) {
        p->M = (uint32_t)(s.n * s.m);
        const uint64_t payload = (uint64_t)s.n * s.m * s.K;
        CHK_RET(EncodeTmap2D(&p->tmapA, heapLocal + wsOff, p->M, s.K, s.K, kBM, kMxBK, 1));
        CHK_RET(EncodeTmap2D(&p->tmapA1, heapLocal + wsOff + half, p->M, s.K, s.K, kBM, kMxBK, 1));
        CHK_RET(EncodeTmap2D(&p->tmapALocal, a, s.m, s.K, s.K, kBM, kMxBK, 1));
        CHK_RET(EncodeTmap2D(&p->tmapB, b, s.N, s.K, s.K, boxB, kMxBK, 1));
        if (pairBN) {
            CHK_RET(EncodeTmapSf(&p->tmapSfA, heapLocal + wsOff + payload, (uint64_t)(p->M / kBM) * kAtoms));
            CHK_RET(EncodeTmapSf(&p->tmapSfA1, heapLocal + wsOff + half + payload, (uint64_t)(p->M / kBM) * kAtoms));
            CHK_RET(EncodeTmapSf(&p->tmapSfALocal, sfa, (uint64_t)((s.m + 127) / 128) * kAtoms));
            CHK_RET(EncodeTmapSf(&p->tmapSfB, sfb, (uint64_t)((s.N + 127) / 128) * kAtoms));
        }
        p->u64[0] = wsOff; p->u64[1] = half; p->u64[2] = (uint64_t)(uintptr_t)a; p->u64[3] = wsOff + payload; p->u64[5] = (uint64_t)(uintptr_t)sfa;
        p->u32[0] = (uint32_t)s.m; p->u32[1] = commCtas; p->u32[2] = (uint32_t)(s.m / kBM);
    } else if (s.kind == MMRS) {
        p->M = (uint32_t)s.m;
        CHK_RET(EncodeTmap2D(&p->tmapA, a, s.m, s.K, s.K, kBM, kMxBK, 1));
        CHK_RET(EncodeTmap2D(&p->tmapB, b, s.N, s.K, s.K, boxB, kMxBK, 1));
        if (pairBN) {
            CHK_RET(EncodeTmapSf(&p->tmapSfA, sfa, (uint64_t)((s.m + 127) / 128) * kAtoms));
            CHK_RET(EncodeTmapSf(&p->tmapSfB, sfb, (uint64_t)((s.N + 127) / 128) * kAtoms));
        }
        p->u64[0] = wsOff; p->u64[1] = half;
        p->u32[0] = (uint32_t)(s.m / s.n); p->u32[1] = (uint32_t)(s.m / s.n / kBM); p->u32[2] = (uint32_t)((s.N + bn - 1) / bn);
    } else {
        const uint32_t colsOwn = (uint32_t)(s.N / s.n);
        p->M = (uint32_t)s.m;
        CHK_RET(EncodeTmap2D(&p->tmapA, a, s.m, s.K, s.K, kBM, kMxBK, 1));
        CHK_RET(EncodeTmap2D(&p->tmapB, b, s.N, s.K, s.K, 128, kMxBK, 1));
        const uint64_t partials = (uint64_t)s.n * s.m * colsOwn * 2, result = (uint64_t)s.m * s.N * 2;
        p->u64[0] = wsOff; p->u64[1] = partials; p->u64[2] = wsOff + 2 * partials; p->u64[3] = result;
        p->u32[0] = colsOwn; p->u32[1] = colsOwn / 128; p->u32[2] = 128;
    }
    return HCCL_SUCCESS;
}

HcclResult BuildParams(const FusedShape &s, char *heapLocal, uint64_t wsOff, const void *a, const void *b, void *out, uint32_t commCtas, GemmParams *p,
                       uint32_t pairBN = 0)
{
    const bool pairMode = pairBN != 0;
    memset(p, 0, sizeof(*p));
    const uint64_t half = WorkspaceHalfBytes(s);
    p->errorWord = GemmErrorWord();
    p->groupM = 16;
    p->outFp32 = 0;
    if (s.kind == AGMM) {
        p->M = (uint32_t)(s.n * s.m); p->N = (uint32_t)s.N; p->K = (uint32_t)s.K; p->ldc = (uint32_t)s.N; p->C = out;
        CHK_RET(EncodeTmap2D(&p->tmapA, heapLocal + wsOff, p->M, s.K, s.K * 2, kBM, kBK, 2));
        CHK_RET(EncodeTmap2D(&p->tmapA1, heapLocal + wsOff + half, p->M, s.K, s.K * 2, kBM, kBK, 2));
        CHK_RET(EncodeTmap2D(&p->tmapALocal, a, s.m, s.K, s.K * 2, kBM, kBK, 2));
        CHK_RET(EncodeTmap2D(&p->tmapB, b, s.N, s.K, s.K * 2, pairMode ? pairBN / 2 : 256, kBK, 2));
        p->u64[0] = wsOff; p->u64[1] = half; p->u64[2] = (uint64_t)(uintptr_t)a;
        p->u32[0] = (uint32_t)s.m; p->u32[1] = commCtas; p->u32[2] = (uint32_t)(s.m / kBM);
        p->u32[3] = pairMode && commCtas == 0 ? 8u : 0u;   // no communication CTAs: spare warps push the shard in 16-row pieces
    } else if (s.kind == MMRS) {
        p->M = (uint32_t)s.m; p->N = (uint32_t)s.N; p->K = (uint32_t)s.K; p->ldc = (uint32_t)s.N; p->C = out;
        CHK_RET(EncodeTmap2D(&p->tmapA, a, s.m, s.K, s.K * 2, kBM, kBK, 2));
        CHK_RET(EncodeTmap2D(&p->tmapB, b, s.N, s.K, s.K * 2, pairMode ? pairBN / 2 : 256, kBK, 2));
        p->u64[0] = wsOff; p->u64[1] = half;
        const uint32_t bn = pairMode ? pairBN : 256;
        p->u32[0] = (uint32_t)(s.m / s.n); p->u32[1] = (uint32_t)(s.m / s.n / kBM); p->u32[2] = (uint32_t)((s.N + bn - 1) / bn);
    } else {
        const uint32_t colsOwn = (uint32_t)(s.N / s.n);
        p->M = (uint32_t)s.m; p->N = (uint32_t)s.N; p->K = (uint32_t)s.K; p->ldc = (uint32_t)s.N; p->C = out;
        CHK_RET(EncodeTmap2D(&p->tmapA, a, s.m, s.K, s.K * 2, kBM, kBK, 2));
        CHK_RET(EncodeTmap2D(&p->tmapB, b, s.N, s.K, s.K * 2, 64, kBK, 2));
        const uint64_t partials = (uint64_t)s.n * s.m * colsOwn * 2, result = (uint64_t)s.m * s.N * 2;
        p->u64[0] = wsOff; p->u64[1] = partials; p->u64[2] = wsOff + 2 * partials; p->u64[3] = result;
        p->u32[0] = colsOwn; p->u32[1] = colsOwn / 64; p->u32[2] = 64;
    }
    return HCCL_SUCCESS;
}

uint32_t GridFor(const FusedShape &s, uint32_t commCtas, uint32_t maxCtas)
{
    uint64_t tiles;
    const uint64_t bn = s.mx ? MxTileN() : 256;
    if (s.kind == AGMM) tiles = (s.n * s.m / kBM) * ((s.N + bn - 1) / bn);
    else if (s.kind == MMRS) tiles = ((s.m + kBM - 1) / kBM) * ((s.N + bn - 1) / bn);
    else tiles = ((s.m + kBM - 1) / kBM) * (s.N / (s.mx ? 128 : 64));
    uint32_t g = (uint32_t)std::min<uint64_t>(tiles + commCtas, maxCtas);
    return std::max(g, commCtas + 1);
}

HcclResult CheckShape(const FusedShape &s)
{
    if (s.K % 8 || s.N % 8 || s.m == 0 || s.N == 0 || s.K == 0) { HCCL_ERROR("fused matmul: K and N must be non-zero multiples of 8"); return HCCL_E_PARA; }
    if (s.kind == AGMM && s.m % kBM) { HCCL_ERROR("AllGatherMatmul: rows per rank (%llu) must be a multiple of 128", (unsigned long long)s.m); return HCCL_E_PARA; }
    if (s.kind == AGMM && s.m / kBM > 64) { HCCL_ERROR("AllGatherMatmul: at most 8192 rows per rank"); return HCCL_E_PARA; }
    if (s.kind == MMRS && (s.m % ((uint64_t)s.n * kBM) || s.m / s.n / kBM > 64)) { HCCL_ERROR("MatmulReduceScatter: M (%llu) must be a multiple of 128 x ranks, at most 8192 rows per rank", (unsigned long long)s.m); return HCCL_E_PARA; }
    if (s.mx && s.K % 128) { HCCL_ERROR("block-scaled fused matmul: K (%llu) must be a multiple of 128", (unsigned long long)s.K); return HCCL_E_PARA; }
    if (s.mx && s.kind == MMAR && (s.N % ((uint64_t)s.n * 128) || ((s.m + kBM - 1) / kBM) * (s.N / s.n / 128) > 64)) {
        HCCL_ERROR("block-scaled MatmulAllReduce: N (%llu) must be a multiple of 128 x ranks", (unsigned long long)s.N);
        return HCCL_E_PARA;
    }
    if (!s.mx && s.kind == MMAR && (s.N % ((uint64_t)s.n * 64) || ((s.m + kBM - 1) / kBM) * (s.N / s.n / 64) > 64)) {
        HCCL_ERROR("MatmulAllReduce: N (%llu) must be a multiple of 64 x ranks and the tiles per owner at most 64", (unsigned long long)s.N);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

template <bool EMU> HcclResult LaunchFused(const FusedShape &s, const GemmParams &p, const GemmParams *devParams, uint32_t grid, uint32_t ranksY, cudaStream_t stream)
{
    const void *fn = nullptr;
    size_t smem = 0;
    if (s.mx && s.kind != MMAR && MxTileN() == 192) {
        if (s.kind == AGMM) { CHK_RET((SetSmemAttrMx<192, AgmmPolicy, EMU>())); fn = (const void *)GemmKernelMx<192, AgmmPolicy, EMU>; }
        else { CHK_RET((SetSmemAttrMx<192, MmrsPolicy, EMU>())); fn = (const void *)GemmKernelMx<192, MmrsPolicy, EMU>; }
        smem = GemmMxSmem<192>::kTotal + 1024;
    } else if (s.mx) {
        if (s.kind == AGMM) { CHK_RET((SetSmemAttrMx<256, AgmmPolicy, EMU>())); fn = (const void *)GemmKernelMx<256, AgmmPolicy, EMU>; smem = GemmMxSmem<256>::kTotal + 1024; }
        else if (s.kind == MMRS) { CHK_RET((SetSmemAttrMx<256, MmrsPolicy, EMU>())); fn = (const void *)GemmKernelMx<256, MmrsPolicy, EMU>; smem = GemmMxSmem<256>::kTotal + 1024; }
        else { CHK_RET((SetSmemAttrMx<128, MmarPolicy, EMU>())); fn = (const void *)GemmKernelMx<128, MmarPolicy, EMU>; smem = GemmMxSmem<128>::kTotal + 1024; }
    } else
    if (s.kind == AGMM) { CHK_RET((SetSmemAttr<256, AgmmPolicy, EMU>())); fn = (const void *)GemmKernel<256, AgmmPolicy, EMU>; smem = GemmSmem<256>::kTotal + 1024; }
    else if (s.kind == MMRS) { CHK_RET((SetSmemAttr<256, MmrsPolicy, EMU>())); fn = (const void *)GemmKernel<256, MmrsPolicy, EMU>; smem = GemmSmem<256>::kTotal + 1024; }
    else { CHK_RET((SetSmemAttr<64, MmarPolicy, EMU>())); fn = (const void *)GemmKernel<64, MmarPolicy, EMU>; smem = GemmSmem<64>::kTotal + 1024; }
    GemmParams pv = p;
    void *args[] = {(void *)&pv, (void *)&devParams};
    cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(grid, ranksY), dim3(kGemmThreads), args, smem, stream);
    if (e != cudaSuccess) { HCCL_ERROR("fused kernel launch failed: %s (grid %u x %u)", cudaGetErrorString(e), grid, ranksY); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

// CTA-pair kernels: clusters of two CTAs, launched cooperatively (every CTA of the op resident) on an even grid.
template <class Policy, int BN> HcclResult LaunchFusedPair(const GemmParams &p, uint32_t grid, cudaStream_t stream)
{
    static std::atomic<bool> attrSet{false};
    auto kern = GemmKernel2Cta<Policy, BN>;
    const size_t smem = Gemm2CtaSmemT<BN>::kTotal + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return HCCL_E_RUNTIME;
        attrSet = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid & ~1u);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) { HCCL_ERROR("fused CTA-pair kernel launch failed: %s (grid %u)", cudaGetErrorString(e), grid); (void)cudaGetLastError(); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

template <class Policy, int BN> HcclResult LaunchFusedPairMx(const GemmParams &p, uint32_t grid, cudaStream_t stream)
{
    static std::atomic<bool> attrSet{false};
    auto kern = GemmKernelMx2Cta<Policy, BN>;
    const size_t smem = GemmMx2CtaSmem<BN>::kTotal + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return HCCL_E_RUNTIME;
        attrSet = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid & ~1u);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) { HCCL_ERROR("fused block-scaled CTA-pair kernel launch failed: %s (grid %u)", cudaGetErrorString(e), grid); (void)cudaGetLastError(); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

// ---- symmetric workspace per communicator (grown on demand; every rank makes the same calls, so offsets agree)
struct ParamKey {
    int kind; const void *a, *b, *out; uint64_t m, N, K, wsOff;     // kind + pair tile width = parameters of the CTA-pair kernel
    const void *sfa = nullptr, *sfb = nullptr;                     // block-scaled operands (kind + 1000)
    bool operator<(const ParamKey &o) const
    {
        return std::tie(kind, a, b, out, m, N, K, wsOff, sfa, sfb) < std::tie(o.kind, o.a, o.b, o.out, o.m, o.N, o.K, o.wsOff, o.sfa, o.sfb);
    }
};
// Encoded tensor maps are reused while the same buffers and shapes come back (decode loops, training steps): encoding four
// maps costs more host time than a decode-sized fused kernel runs.
struct Workspace { void *ptr = nullptr; uint64_t bytes = 0; std::map<ParamKey, GemmParams> params; };
std::mutex g_wsMu;
std::map<Comm *, Workspace> g_ws;

HcclResult EnsureWorkspace(Comm *c, uint64_t bytes, uint64_t *off)
{
    std::lock_guard<std::mutex> lk(g_wsMu);
    Workspace &w = g_ws[c];
    if (w.bytes < bytes) {
        if (w.ptr) {
            // the old window may still be in use by kernels in flight on this or a peer rank
            cudaDeviceSynchronize();
            CHK_RET(c->boot->Barrier());
            SymFree(c, w.ptr);
            w.ptr = nullptr;
            w.bytes = 0;
            w.params.clear();
        }
        uint64_t want = (bytes + (1 << 20) - 1) & ~((1ull << 20) - 1);
        CHK_RET(SymAlloc(c, want, &w.ptr));
        w.bytes = want;
    }
    *off = SymOffsetOf(c, w.ptr);
    return HCCL_SUCCESS;
}

// copies the gathered activations of the op that just ran (parity = opCount - 1) into a user buffer
__global__ void CopyGatheredKernel(const DevComm *c, uint64_t gatherOff, uint64_t halfBytes, const char *aLocal, char *dst, uint64_t shardBytes)
{
    char *heap = c->heap[c->rank];
    uint32_t half = (CtrlOf(heap)->opCount - 1u) & 1u;
    const char *src = heap + gatherOff + (uint64_t)half * halfBytes;
    for (int r = 0; r < c->nranks; ++r) {
        dev::Part p = dev::PartOf(shardBytes, gridDim.x, blockIdx.x);
        const char *from = r == c->rank ? aLocal : src + (uint64_t)r * shardBytes;
        dev::BlockCopy(dst + (uint64_t)r * shardBytes + p.off, from + p.off, p.len);
    }
}

}  // namespace

void DropWorkspace(Comm *c)
{
    std::lock_guard<std::mutex> lk(g_wsMu);
    g_ws.erase(c);
}

HcclResult RunFused(FusedKind kind, Comm *c, const void *a, const void *b, void *out, void *gathered, uint64_t m, uint64_t N, uint64_t K, cudaStream_t stream,
                    const void *sfa = nullptr, const void *sfb = nullptr)
{
    CHK_RET(CommCheckReady(c));
    if (c->backend != BackendKind::CUDA) { HCCL_ERROR("fused matmul operators need a CUDA communicator"); return HCCL_E_NOT_SUPPORT; }
    FusedShape s{kind, c->nranks, c->rank, m, N, K, sfa != nullptr};
    CHK_RET(CheckShape(s));
    uint64_t wsOff = 0;
    CHK_RET(EnsureWorkspace(c, 2 * WorkspaceHalfBytes(s) + 4096, &wsOff));
    const bool pairMode = PairModeFor(s);
    uint32_t commCtas = kind == AGMM && !(pairMode && PairLevel() >= 3) ? CommCtasDefault() : 0;
    if (pairMode) commCtas &= ~1u;                       // whole CTA pairs take the communication role
    const uint32_t pairs = ((uint32_t)SmCount() - commCtas) / 2;
    const uint64_t rowPairs = kind == AGMM ? s.n * s.m / kBM / 2 : s.m / kBM / 2;
    // block-scaled pairs: 192-wide tiles (two accumulators) unless K is long enough to hide the epilogue of 256-wide ones
    const uint32_t pairBN = !pairMode ? 0 : s.mx ? (s.K >= 16384 ? 256u : 192u) : PairTileN(rowPairs, s.N, pairs);
    GemmParams p;
    {
        std::lock_guard<std::mutex> lk(g_wsMu);
        auto &cache = g_ws[c].params;
        ParamKey key{(int)kind + (int)pairBN + (s.mx ? 1000 + (int)MxTileN() : 0), a, b, out, m, N, K, wsOff, sfa, sfb};
        auto it = cache.find(key);
        if (it != cache.end()) p = it->second;
        else {
            if (s.mx) CHK_RET(BuildParamsMx(s, c->heap[c->rank], wsOff, a, sfa, b, sfb, out, commCtas, &p, pairBN));
            else CHK_RET(BuildParams(s, c->heap[c->rank], wsOff, a, b, out, commCtas, &p, pairBN));
            p.comm = c->devCommPtr;
            if (cache.size() > 256) cache.clear();
            cache[key] = p;
        }
    }
    if (pairMode) {
        uint64_t pairTiles = rowPairs * ((s.N + pairBN - 1) / pairBN);
        uint32_t grid = (uint32_t)std::min<uint64_t>(pairTiles * 2, (uint64_t)pairs * 2) + commCtas;
        grid = std::max(grid, commCtas + 2u);
        if (s.mx && kind == AGMM && pairBN == 192) CHK_RET((LaunchFusedPairMx<AgmmPolicy, 192>(p, grid, stream)));
        else if (s.mx && kind == AGMM) CHK_RET((LaunchFusedPairMx<AgmmPolicy, 256>(p, grid, stream)));
        else if (s.mx && pairBN == 192) CHK_RET((LaunchFusedPairMx<MmrsPolicy, 192>(p, grid, stream)));
        else if (s.mx) CHK_RET((LaunchFusedPairMx<MmrsPolicy, 256>(p, grid, stream)));
        else if (kind == AGMM && pairBN == 224) CHK_RET((LaunchFusedPair<AgmmPolicy, 224>(p, grid, stream)));
        else if (kind == AGMM) CHK_RET((LaunchFusedPair<AgmmPolicy, 256>(p, grid, stream)));
        else if (pairBN == 224) CHK_RET((LaunchFusedPair<MmrsPolicy, 224>(p, grid, stream)));
        else CHK_RET((LaunchFusedPair<MmrsPolicy, 256>(p, grid, stream)));
    } else {
        uint32_t grid = GridFor(s, commCtas, (uint32_t)SmCount());
        CHK_RET(LaunchFused<false>(s, p, nullptr, grid, 1, stream));
    }
    c->counters.kernelsLaunched++;
    c->devOpIssued++;
    CountLaunch();
    c->counters.ops++;
    if (kind == AGMM && gathered && !s.mx) {
        CopyGatheredKernel<<<32, 512, 0, stream>>>(c->devCommPtr, wsOff, WorkspaceHalfBytes(s), (const char *)a, (char *)gathered, m * K * 2);
        if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace mc2
}  // namespace hccl

using namespace hccl;
using namespace hccl::mc2;

extern "C" {

HcclResult HcclAllGatherMatmul(const void *aLocal, const void *b, void *out, void *gathered, uint64_t mLocal, uint64_t n, uint64_t k,
                               HcclDataType dataType, HcclComm comm, cudaStream_t stream)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!aLocal || !b || !out) { HCCL_ERROR("[EI0003] HcclAllGatherMatmul: null buffer"); return HCCL_E_PTR; }
    if (dataType != HCCL_DATA_TYPE_BFP16) { HCCL_ERROR("HcclAllGatherMatmul supports bf16 (got %s)", DataTypeName(dataType)); return HCCL_E_NOT_SUPPORT; }
    if (c->nranks == 1) {
        if (gathered && gathered != aLocal) CHK_RET(LocalCopyAsync(c, gathered, aLocal, mLocal * k * 2, stream));
        return HcclGemmBf16(aLocal, b, out, mLocal, n, k, 0, stream);
    }
    return RunFused(AGMM, c, aLocal, b, out, gathered, mLocal, n, k, stream);
}

HcclResult HcclMatmulReduceScatter(const void *a, const void *b, void *out, uint64_t m, uint64_t n, uint64_t kLocal, HcclDataType dataType,
                                   HcclComm comm, cudaStream_t stream)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!a || !b || !out) { HCCL_ERROR("[EI0003] HcclMatmulReduceScatter: null buffer"); return HCCL_E_PTR; }
    if (dataType != HCCL_DATA_TYPE_BFP16) return HCCL_E_NOT_SUPPORT;
    if (c->nranks == 1) return HcclGemmBf16(a, b, out, m, n, kLocal, 0, stream);
    return RunFused(MMRS, c, a, b, out, nullptr, m, n, kLocal, stream);
}

HcclResult HcclMatmulAllReduce(const void *a, const void *b, void *out, uint64_t m, uint64_t n, uint64_t kLocal, HcclDataType dataType,
                               HcclComm comm, cudaStream_t stream)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!a || !b || !out) { HCCL_ERROR("[EI0003] HcclMatmulAllReduce: null buffer"); return HCCL_E_PTR; }
    if (dataType != HCCL_DATA_TYPE_BFP16) return HCCL_E_NOT_SUPPORT;
    if (c->nranks == 1) return HcclGemmBf16(a, b, out, m, n, kLocal, 0, stream);
    return RunFused(MMAR, c, a, b, out, nullptr, m, n, kLocal, stream);
}

// ---- block-scaled (MXFP8) forms: e4m3 payloads with e8m0 scale atoms as written by HcclQuantizeMxfp8; bf16 results.
HcclResult HcclAllGatherMatmulMxfp8(const void *aLocal, const void *sfaLocal, const void *b, const void *sfb, void *out, uint64_t mLocal, uint64_t n,
                                    uint64_t k, HcclComm comm, cudaStream_t stream)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!aLocal || !sfaLocal || !b || !sfb || !out) { HCCL_ERROR("[EI0003] HcclAllGatherMatmulMxfp8: null buffer"); return HCCL_E_PTR; }
    if (c->nranks == 1) return HcclGemmMxfp8(aLocal, sfaLocal, b, sfb, out, mLocal, n, k, 0, stream);
    return RunFused(AGMM, c, aLocal, b, out, nullptr, mLocal, n, k, stream, sfaLocal, sfb);
}

HcclResult HcclMatmulReduceScatterMxfp8(const void *a, const void *sfa, const void *b, const void *sfb, void *out, uint64_t m, uint64_t n, uint64_t kLocal,
                                        HcclComm comm, cudaStream_t stream)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!a || !sfa || !b || !sfb || !out) { HCCL_ERROR("[EI0003] HcclMatmulReduceScatterMxfp8: null buffer"); return HCCL_E_PTR; }
    if (c->nranks == 1) return HcclGemmMxfp8(a, sfa, b, sfb, out, m, n, kLocal, 0, stream);
    return RunFused(MMRS, c, a, b, out, nullptr, m, n, kLocal, stream, sfa, sfb);
}

HcclResult HcclMatmulAllReduceMxfp8(const void *a, const void *sfa, const void *b, const void *sfb, void *out, uint64_t m, uint64_t n, uint64_t kLocal,
                                    HcclComm comm, cudaStream_t stream)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!a || !sfa || !b || !sfb || !out) { HCCL_ERROR("[EI0003] HcclMatmulAllReduceMxfp8: null buffer"); return HCCL_E_PTR; }
    if (c->nranks == 1) return HcclGemmMxfp8(a, sfa, b, sfb, out, m, n, kLocal, 0, stream);
    return RunFused(MMAR, c, a, b, out, nullptr, m, n, kLocal, stream, sfa, sfb);
}

// Emulation of the block-scaled forms (same conventions as HcclEmuFusedRun; sfas / sfbs: per-rank scale atoms).
HcclResult HcclEmuFusedRunMx(void *emu, int kind, void **as, void **sfas, void **bs, void **sfbs, void **outs, uint64_t m, uint64_t n, uint64_t k,
                             uint32_t ctasPerRank, uint32_t commCtas)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !as || !sfas || !bs || !sfbs || !outs) return HCCL_E_PTR;
    uint32_t R = (uint32_t)w->nranks;
    std::vector<GemmParams> ps(R);
    FusedShape s0{(FusedKind)kind, R, 0, m, n, k, true};
    CHK_RET(CheckShape(s0));
    if (2 * WorkspaceHalfBytes(s0) + 4096 > w->arenaBytes) { HCCL_ERROR("emu arena too small: need %llu", (unsigned long long)(2 * WorkspaceHalfBytes(s0) + 4096)); return HCCL_E_MEMORY; }
    if (kind != AGMM) commCtas = 0;
    for (uint32_t r = 0; r < R; ++r) {
        FusedShape s{(FusedKind)kind, R, r, m, n, k, true};
        CHK_RET(BuildParamsMx(s, w->heaps[r], w->arenaOff, as[r], sfas[r], bs[r], sfbs[r], outs[r], commCtas, &ps[r]));
        ps[r].comm = w->devComms + r;
    }
    if (sizeof(GemmParams) > 2048) return HCCL_E_INTERNAL;
    if (cudaMemcpy(w->devFusedParams, ps.data(), sizeof(GemmParams) * R, cudaMemcpyHostToDevice) != cudaSuccess) return HCCL_E_RUNTIME;
    uint32_t grid = std::max(ctasPerRank, commCtas + 1);
    CHK_RET(LaunchFused<true>(s0, ps[0], (const GemmParams *)w->devFusedParams, grid, R, 0));
    if (cudaStreamSynchronize(0) != cudaSuccess) { HCCL_ERROR("emu fused kernel failed: %s", cudaGetErrorString(cudaGetLastError())); return HCCL_E_RUNTIME; }
    for (uint32_t r = 0; r < R; ++r) if (w->status[r].code != 0) return HCCL_E_TIMEOUT;
    return GemmCheckError();
}

// Emulation: kind 0 AllGatherMatmul (m = rows per rank), 1 MatmulReduceScatter, 2 MatmulAllReduce. as/bs/outs: per-rank
// device pointers. ctasPerRank * nranks must fit on the GPU (one CTA per SM).
HcclResult HcclEmuFusedRun(void *emu, int kind, void **as, void **bs, void **outs, uint64_t m, uint64_t n, uint64_t k, uint32_t ctasPerRank, uint32_t commCtas)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !as || !bs || !outs) return HCCL_E_PTR;
    uint32_t R = (uint32_t)w->nranks;
    std::vector<GemmParams> ps(R);
    FusedShape s0{(FusedKind)kind, R, 0, m, n, k};
    CHK_RET(CheckShape(s0));
    if (2 * WorkspaceHalfBytes(s0) + 4096 > w->arenaBytes) { HCCL_ERROR("emu arena too small: need %llu", (unsigned long long)(2 * WorkspaceHalfBytes(s0) + 4096)); return HCCL_E_MEMORY; }
    if (kind != AGMM) commCtas = 0;
    for (uint32_t r = 0; r < R; ++r) {
        FusedShape s{(FusedKind)kind, R, r, m, n, k};
        CHK_RET(BuildParams(s, w->heaps[r], w->arenaOff, as[r], bs[r], outs[r], commCtas, &ps[r]));
        ps[r].comm = w->devComms + r;
    }
    if (sizeof(GemmParams) > 2048) return HCCL_E_INTERNAL;
    if (cudaMemcpy(w->devFusedParams, ps.data(), sizeof(GemmParams) * R, cudaMemcpyHostToDevice) != cudaSuccess) return HCCL_E_RUNTIME;
    uint32_t grid = std::max(ctasPerRank, commCtas + 1);
    CHK_RET(LaunchFused<true>(s0, ps[0], (const GemmParams *)w->devFusedParams, grid, R, 0));
    if (cudaStreamSynchronize(0) != cudaSuccess) { HCCL_ERROR("emu fused kernel failed: %s", cudaGetErrorString(cudaGetLastError())); return HCCL_E_RUNTIME; }
    for (uint32_t r = 0; r < R; ++r) if (w->status[r].code != 0) return HCCL_E_TIMEOUT;
    return GemmCheckError();
}

}  // extern "C"
