// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (both operands K-major, bf16 in,
// fp32 accumulate in tensor memory, bf16 or fp32 out).
//
//   warp 0   TMA producer: streams 128xBK A tiles and BNxBK B tiles into a STAGES-deep shared-memory ring
//   warp 1   MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM accumulators
//   warp 2   owns the TMEM allocation
//   warps 4-7 epilogue: tcgen05.ld the finished accumulator (each warp its own 32-lane quarter), convert, store
// The two accumulators let the epilogue of tile i overlap the main loop of tile i+1. The kernel is persistent: one CTA
// per SM walks tiles in an L2-friendly grouped order.
//
// The collective fusions reuse this skeleton through a Policy type:
//   Policy::TileCoord(p, linearTile, &mBlk, &nBlk)    tile order (e.g. local rows first for AllGather+matmul)
//   Policy::WaitRowsReady(p, mBlk, abortWord)         producer-side gate before loading A rows (gathered rows landed?)
//   Policy::Store(p, row, col0, v[32], lane info)     epilogue sink (local C, a peer's reduce-scatter slot, ...)
//   Policy::TileDone(p, mBlk, nBlk)                   after a tile's stores (signal the consumer rank)
// HCCL has no counterpart: its MC2 header only hands a communication context to external fused kernels (reference:
// include/hccl_mc2.h:25-82, src/common/hccl_mc2.cc:141-165); the kernels themselves are new here.
#pragma once
#include <cuda_bf16.h>
#include "sm100_ptx.cuh"

namespace hccl {
namespace mc2 {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int kGemmThreads = 256;

struct GemmParams {
    CUtensorMap tmapA;           // [M, K] bf16, box 64 x 128, 128B swizzle
    CUtensorMap tmapB;           // [N, K] bf16, box 64 x BN
    void *C;                     // output, row-major, leading dimension ldc (elements)
    uint32_t M, N, K;
    uint32_t ldc;
    uint32_t outFp32;            // 1 = fp32 output
    uint32_t groupM;             // M blocks per rasterisation group
    uint32_t *errorWord;         // device word set to 1 when a wait ran out
    // fusion fields (meaning defined by the policy)
    const void *comm;            // DevComm*
    uint64_t u64[8];
    uint32_t u32[8];
};

template <int BN> struct GemmSmem {
    static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kRing = kStages * (kABytes + kBBytes);
    static constexpr int kBarOff = kRing;
    static constexpr int kTotal = kRing + 256;
};

struct PlainPolicy {
    __device__ static void TileCoord(const GemmParams &p, uint32_t t, uint32_t mBlocks, uint32_t nBlocks, uint32_t *mb, uint32_t *nb)
    {
        // grouped rasterisation: walk groupM row-blocks down, then move one column-block right
        uint32_t g = p.groupM ? p.groupM : 16;
        uint32_t perGroup = g * nBlocks;
        uint32_t group = t / perGroup;
        uint32_t first = group * g;
        uint32_t size = mBlocks - first < g ? mBlocks - first : g;
        uint32_t in = t % perGroup;
        *mb = first + in % size;
        *nb = in / size;
    }
    __device__ static bool WaitRowsReady(const GemmParams &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void Store(const GemmParams &p, uint32_t row, uint32_t col0, const uint32_t (&v)[32])
    {
        if (row >= p.M) return;
        if (p.outFp32) {
            float *c = (float *)p.C + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                if (col0 + j < p.N) *(uint4 *)(c + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        } else {
            __nv_bfloat16 *c = (__nv_bfloat16 *)p.C + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                if (col0 + j < p.N) {
                    uint4 o;
                    __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                    __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                    __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                    o.x = *(uint32_t *)&t0; o.y = *(uint32_t *)&t1; o.z = *(uint32_t *)&t2; o.w = *(uint32_t *)&t3;
                    *(uint4 *)(c + j) = o;
                }
            }
        }
    }
    __device__ static void TileDone(const GemmParams &, uint32_t, uint32_t, uint32_t) {}
};

template <int BN, class Policy>
__global__ void __launch_bounds__(kGemmThreads, 1) GemmKernel(const __grid_constant__ GemmParams p)
{
    using S = GemmSmem<BN>;
    constexpr int STAGES = S::kStages;
    constexpr uint32_t kTmemCols = BN * 2 >= 32 ? BN * 2 : 32;       // two accumulators
    constexpr uint32_t kIdesc = MakeInstrDesc(FMT_BF16, FMT_BF16, kBM, BN);
    extern __shared__ uint8_t smemRaw[];
    // 1024-byte alignment for the swizzle atoms
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem;
    uint8_t *sB = smem + STAGES * S::kABytes;
    uint64_t *full = (uint64_t *)(smem + S::kBarOff);
    uint64_t *empty = full + STAGES;
    uint64_t *tmemFull = empty + STAGES;
    uint64_t *tmemEmpty = tmemFull + 2;
    uint32_t *tmemPtr = (uint32_t *)(tmemEmpty + 2);
    volatile uint32_t *abortWord = (volatile uint32_t *)(tmemPtr + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t mBlocks = (p.M + kBM - 1) / kBM, nBlocks = (p.N + BN - 1) / BN;
    const uint32_t numTiles = mBlocks * nBlocks;
    const uint32_t kIters = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { MbarInit(&tmemFull[s], 1); MbarInit(&tmemEmpty[s], 128); }
        *abortWord = 0;
        MbarInitFence();
        PrefetchTmap(&p.tmapA);
        PrefetchTmap(&p.tmapB);
    }
    if (warp == 2) { TmemAlloc(tmemPtr, kTmemCols); TmemRelinquish(); }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmemBase = *tmemPtr;

    if (warp == 0) {
        if (ElectOne()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                uint32_t mb, nb;
                Policy::TileCoord(p, t, mBlocks, nBlocks, &mb, &nb);
                ok = Policy::WaitRowsReady(p, mb, abortWord);
                for (uint32_t kb = 0; kb < kIters && ok; ++kb) {
                    ok = MbarWait(&empty[stage], phase ^ 1, abortWord);
                    if (!ok) break;
                    MbarExpectTx(&full[stage], S::kABytes + S::kBBytes);
                    TmaLoad2D(sA + stage * S::kABytes, &p.tmapA, &full[stage], (int32_t)(kb * kBK), (int32_t)(mb * kBM));
                    TmaLoad2D(sB + stage * S::kBBytes, &p.tmapB, &full[stage], (int32_t)(kb * kBK), (int32_t)(nb * BN));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (ElectOne()) {
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                ok = MbarWait(&tmemEmpty[acc], accPhase ^ 1, abortWord);
                if (!ok) break;
                TcFenceAfter();
                const uint32_t dTmem = tmemBase + acc * BN;
                for (uint32_t kb = 0; kb < kIters; ++kb) {
                    ok = MbarWait(&full[stage], phase, abortWord);
                    if (!ok) break;
                    TcFenceAfter();
                    uint64_t aDesc = MakeSmemDescSw128(SmemAddr(sA + stage * S::kABytes));
                    uint64_t bDesc = MakeSmemDescSw128(SmemAddr(sB + stage * S::kBBytes));
#pragma unroll
                    for (uint32_t k = 0; k < kBK / 16; ++k)
                        UmmaF16(dTmem, AdvanceDescK(aDesc, k * 32), AdvanceDescK(bDesc, k * 32), kIdesc, (kb | k) != 0 ? 1u : 0u);
                    UmmaCommit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                UmmaCommit(&tmemFull[acc]);
                acc ^= 1;
                if (acc == 0) accPhase ^= 1;
            }
        }
    } else if (warp >= 4) {
        const uint32_t ew = warp - 4;
        uint32_t acc = 0, accPhase = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
            uint32_t mb, nb;
            Policy::TileCoord(p, t, mBlocks, nBlocks, &mb, &nb);
            ok = MbarWait(&tmemFull[acc], accPhase, abortWord);
            if (!ok) break;
            TcFenceAfter();
            const uint32_t row = mb * kBM + ew * 32 + lane;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                TmemLd32x32(tmemBase + ((ew * 32) << 16) + acc * BN + c * 32, v);
                TmemLdWait();
                Policy::Store(p, row, nb * BN + c * 32, v);
            }
            TcFenceBefore();
            MbarArrive(&tmemEmpty[acc]);
            Policy::TileDone(p, mb, nb, ew);
            acc ^= 1;
            if (acc == 0) accPhase ^= 1;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abortWord != 0 && p.errorWord) *p.errorWord = 1;
    if (warp == 2) { TcFenceAfter(); TmemDealloc(tmemBase, kTmemCols); }
}

}  // namespace mc2
}  // namespace hccl
