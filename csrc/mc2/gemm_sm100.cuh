// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (both operands K-major, bf16 in,
// fp32 accumulate in tensor memory, bf16 or fp32 out), and the skeleton the fused matmul+collective kernels share.
//
//   warp 0   TMA producer: streams 128xBK A tiles and BNxBK B tiles into a STAGES-deep shared-memory ring
//   warp 1   MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM accumulators
//   warp 2   owns the TMEM allocation
//   warps 4-7 epilogue: tcgen05.ld the finished accumulator (each warp its own 32-lane quarter), convert, store
// The two accumulators let the epilogue of tile i overlap the main loop of tile i+1. The kernel is persistent: one CTA
// per SM walks tiles in an L2-friendly order.
//
// A Policy type customises the skeleton (all hooks are static device functions):
//   Init(p, ctx)                         per-CTA context (rank, op parity, ...)
//   CommCtas(p)                          leading CTAs that run CommRole instead of GEMM tiles
//   CommRole(p, ctx, smem)               e.g. push the local activation shard to every peer with bulk copies
//   TileCoord(p, ctx, t, mBlocks, nBlocks, &mb, &nb)   tile order
//   WaitRowsReady(p, ctx, mb, abort)     producer-side gate before loading A rows
//   SelectA(p, ctx, mb, &tmap, &row)     which tensor map / row coordinate serves this row block
//   Store(p, ctx, row, col0, v[32])      epilogue sink (local C, a peer's reduce-scatter slot, ...)
//   EpilogueGate / Combine               per-tile gate and per-chunk transform of the accumulator (add received partials)
//   TileDone(p, ctx, mb, nb, ew, lane)   after a tile's stores (signal the consumer rank)
//   PostPhase(p, ctx, cta, ctas, abort)  work after the last tile (ordered reduction of the received partials)
//   Exit(p, ctx)                         per-CTA exit protocol
// EMU = true: several ranks share the GPU, blockIdx.y is the rank and parameters come from an array in device memory
// (cooperative launch; used by the single-GPU tests).
// HCCL has no counterpart of these kernels: its MC2 header only hands a communication context to external fused
// kernels (reference: include/hccl_mc2.h:25-82, src/common/hccl_mc2.cc:141-165).
#pragma once
#include <cuda_bf16.h>
#include "sm100_ptx.cuh"

// Debug flavor: stores through peer pointers are range-checked when the including file brought the collective primitives in
// (the fused operators); the plain GEMM writes only caller memory.
#ifndef HCCL_RANGE_OK
#define HCCL_RANGE_OK(p, n) true
#endif

namespace hccl {
namespace mc2 {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int kGemmThreads = 256;

struct GemmParams {
    CUtensorMap tmapA;           // [M, K] bf16, box 64 x 128, 128B swizzle
    CUtensorMap tmapA1;          // policy-specific second A map (other parity half)
    CUtensorMap tmapALocal;      // policy-specific third A map (the local shard)
    CUtensorMap tmapB;           // [N, K] bf16, box 64 x BN
    CUtensorMap tmapSfA, tmapSfB; // block-scaled CTA-pair kernel: scale atoms as [atoms][128 x u32] (box = one atom, no swizzle)
    CUtensorMap tmapSfA1, tmapSfALocal;   // policy-specific further scale maps of A (other parity half, the local shard)
    void *C;                     // output, row-major, leading dimension ldc (elements)
    uint32_t M, N, K;
    uint32_t ldc;
    uint32_t outFp32;            // 1 = fp32 output
    uint32_t groupM;             // M blocks per rasterisation group
    uint32_t waitSleepNs;        // back-off of the off-critical-path barrier waits (0 = spin)
    uint32_t *errorWord;         // device word set to 1 when a wait ran out
    const void *comm;            // DevComm* of this rank (fused policies)
    uint64_t u64[8];
    uint32_t u32[8];
    // block-scaled (MXFP8) kernels: e8m0 scale atoms of A and B, [rows / 128][K / 128][512 bytes]
    const uint8_t *sfA;
    const uint8_t *sfB;
    uint32_t sfAtomsB;           // 128-row atoms B's scale array holds along N
    uint32_t elemBytes;          // operand element size (0 or 2 = bf16, 1 = fp8)
    uint32_t waitHintNs;         // suspend-time hint of the barrier waits (0 = plain polling)
    uint32_t epiSleepNs;         // CTA-pair kernel: back-off of the epilogue's wait for a finished accumulator
};

template <int BN> struct GemmSmem {
    static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kRing = kStages * (kABytes + kBBytes);
    static constexpr int kStageCols = BN < 128 ? BN : 128;                 // columns staged per epilogue pass
    static constexpr int kStagingOff = kRing;
    static constexpr int kStagingBytes = kBM * kStageCols * 2;             // bf16 tile slice, XOR-swizzled 16-byte chunks
    static constexpr int kBarOff = kRing + kStagingBytes;
    static constexpr int kTotal = kBarOff + 256;
};

__device__ __forceinline__ void StoreRow32(void *C, uint32_t ldc, uint32_t N, bool fp32, uint32_t row, uint32_t col0, const uint32_t (&v)[32])
{
    if (fp32) {
        float *c = (float *)C + (size_t)row * ldc + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            if (col0 + j < N) *(uint4 *)(c + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
        __nv_bfloat16 *c = (__nv_bfloat16 *)C + (size_t)row * ldc + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            if (col0 + j < N) {
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

struct PlainPolicy {
    struct Ctx {};
    __device__ static void Init(const GemmParams &, Ctx &) {}
    __device__ static uint32_t CommCtas(const GemmParams &) { return 0; }
    __device__ static void CommRole(const GemmParams &, Ctx &, uint8_t *) {}
    __device__ static void TileCoord(const GemmParams &p, const Ctx &, uint32_t t, uint32_t mBlocks, uint32_t nBlocks, uint32_t *mb, uint32_t *nb)
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
    // CTA-pair kernel: the same order over 256-row block pairs
    __device__ static void TileCoordPairs(const GemmParams &p, const Ctx &c, uint32_t t, uint32_t mPairs, uint32_t nBlocks, uint32_t *mb2, uint32_t *nb)
    {
        TileCoord(p, c, t, mPairs, nBlocks, mb2, nb);
    }
    __device__ static void SpareWarps(const GemmParams &, Ctx &, uint32_t, uint32_t, uint32_t, uint32_t, volatile uint32_t *) {}
    __device__ static bool WaitRowsReady(const GemmParams &, const Ctx &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void SelectA(const GemmParams &p, const Ctx &, uint32_t mb, const CUtensorMap **tm, int32_t *row)
    {
        *tm = &p.tmapA;
        *row = (int32_t)(mb * kBM);
    }
    // block-scaled kernels: the scale atoms (512 bytes per 128 rows x 128 K) of row block mb, K block 0
    __device__ static const uint8_t *SelectSfA(const GemmParams &p, const Ctx &, uint32_t mb) { return p.sfA + (uint64_t)mb * (p.K / 128) * 512; }
    // the same for the kernel that fetches scale atoms through a tensor map: map and atom row of K block 0
    __device__ static void SelectSfAMap(const GemmParams &p, const Ctx &, uint32_t mb, const CUtensorMap **tm, int32_t *atomRow)
    {
        *tm = &p.tmapSfA;
        *atomRow = (int32_t)(mb * (p.K / 128));
    }
    // fp32 output goes straight from registers; bf16 output is staged through shared memory and written as whole
    // 16-byte chunks of contiguous row segments
    __device__ static bool UseDirect(const GemmParams &p) { return p.outFp32 != 0; }
    __device__ static void Store(const GemmParams &p, const Ctx &, uint32_t row, uint32_t col0, const uint32_t (&v)[32])
    {
        if (row < p.M) StoreRow32(p.C, p.ldc, p.N, p.outFp32 != 0, row, col0, v);
    }
    // destination of 8 consecutive bf16 results at (row, col), or nullptr when outside the output
    __device__ static __nv_bfloat16 *RowDst(const GemmParams &p, const Ctx &, uint32_t row, uint32_t col)
    {
        return (row < p.M && col < p.N) ? (__nv_bfloat16 *)p.C + (size_t)row * p.ldc + col : nullptr;
    }
    // called by all 128 epilogue threads before a tile's accumulator is read / for every 32-column chunk read
    __device__ static bool EpilogueGate(const GemmParams &, Ctx &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void Combine(const GemmParams &, const Ctx &, uint32_t, uint32_t, uint32_t, uint32_t (&)[32]) {}
    __device__ static void TileDone(const GemmParams &, const Ctx &, uint32_t, uint32_t, uint32_t, uint32_t) {}
    __device__ static void PostPhase(const GemmParams &, Ctx &, uint32_t, uint32_t, volatile uint32_t *) {}
    __device__ static void Exit(const GemmParams &, Ctx &) {}
};

template <int BN, class Policy, bool EMU>
__global__ void __launch_bounds__(kGemmThreads, 1) GemmKernel(const __grid_constant__ GemmParams pv, const GemmParams *emuParams)
{
    const GemmParams &p = EMU ? emuParams[blockIdx.y] : pv;
    using S = GemmSmem<BN>;
    constexpr int STAGES = S::kStages;
    constexpr uint32_t kTmemCols = BN * 2 >= 32 ? BN * 2 : 32;       // two accumulators
    constexpr uint32_t kIdesc = MakeInstrDesc(FMT_BF16, FMT_BF16, kBM, BN);
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);   // swizzle atoms want 1024-byte alignment

    typename Policy::Ctx ctx;
    Policy::Init(p, ctx);
    const uint32_t commCtas = Policy::CommCtas(p);
    if (blockIdx.x < commCtas) {
        Policy::CommRole(p, ctx, smem);
        Policy::Exit(p, ctx);
        return;
    }
    const uint32_t cta = blockIdx.x - commCtas, ctas = gridDim.x - commCtas;

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
            for (uint32_t t = cta; t < numTiles && ok; t += ctas) {
                uint32_t mb, nb;
                Policy::TileCoord(p, ctx, t, mBlocks, nBlocks, &mb, &nb);
                ok = Policy::WaitRowsReady(p, ctx, mb, abortWord);
                const CUtensorMap *ta;
                int32_t rowA;
                Policy::SelectA(p, ctx, mb, &ta, &rowA);
                for (uint32_t kb = 0; kb < kIters && ok; ++kb) {
                    ok = MbarWaitRelaxed(&empty[stage], phase ^ 1, abortWord, p.waitSleepNs);
                    if (!ok) break;
                    MbarExpectTx(&full[stage], S::kABytes + S::kBBytes);
                    TmaLoad2D(sA + stage * S::kABytes, ta, &full[stage], (int32_t)(kb * kBK), rowA);
                    TmaLoad2D(sB + stage * S::kBBytes, &p.tmapB, &full[stage], (int32_t)(kb * kBK), (int32_t)(nb * BN));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (ElectOne()) {
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t t = cta; t < numTiles && ok; t += ctas) {
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
        for (uint32_t t = cta; t < numTiles && ok; t += ctas) {
            uint32_t mb, nb;
            Policy::TileCoord(p, ctx, t, mBlocks, nBlocks, &mb, &nb);
            ok = MbarWaitRelaxed(&tmemFull[acc], accPhase, abortWord, p.waitSleepNs);
            if (!ok) break;
            TcFenceAfter();
            const uint32_t rowInTile = ew * 32 + lane;
            const uint32_t row = mb * kBM + rowInTile;
            if (Policy::UseDirect(p)) {
#pragma unroll 1
                for (uint32_t c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    TmemLd32x32(tmemBase + ((ew * 32) << 16) + acc * BN + c * 32, v);
                    TmemLdWait();
                    Policy::Store(p, ctx, row, nb * BN + c * 32, v);
                }
                TcFenceBefore();
                MbarArrive(&tmemEmpty[acc]);
            } else {
                constexpr uint32_t SC = S::kStageCols, CH = SC / 8;          // staged columns / 16-byte chunks per row
                uint4 *stg = (uint4 *)(smem + S::kStagingOff);
                const uint32_t et = threadIdx.x - 128;                       // 0..127 among the epilogue threads
                if (!Policy::EpilogueGate(p, ctx, mb, abortWord)) { ok = false; break; }
#pragma unroll 1
                for (uint32_t pass = 0; pass < BN / SC; ++pass) {
#pragma unroll 1
                    for (uint32_t c = 0; c < SC / 32; ++c) {
                        uint32_t v[32];
                        TmemLd32x32(tmemBase + ((ew * 32) << 16) + acc * BN + pass * SC + c * 32, v);
                        TmemLdWait();
                        Policy::Combine(p, ctx, mb, row, nb * BN + pass * SC + c * 32, v);
#pragma unroll
                        for (uint32_t q = 0; q < 4; ++q) {
                            uint4 o;
                            __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
                            __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
                            __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
                            o.x = *(uint32_t *)&t0; o.y = *(uint32_t *)&t1; o.z = *(uint32_t *)&t2; o.w = *(uint32_t *)&t3;
                            stg[rowInTile * CH + ((c * 4 + q) ^ (rowInTile & 7))] = o;
                        }
                    }
                    if (pass + 1 == BN / SC) {                               // accumulator fully read: hand it back early
                        TcFenceBefore();
                        MbarArrive(&tmemEmpty[acc]);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 4
                    for (uint32_t i = et; i < (uint32_t)kBM * CH; i += 128) {
                        const uint32_t r = i / CH, ch = i % CH;
                        __nv_bfloat16 *dst = Policy::RowDst(p, ctx, mb * kBM + r, nb * BN + pass * SC + ch * 8);
                        if (dst && HCCL_RANGE_OK(dst, 16)) *(uint4 *)dst = stg[r * CH + (ch ^ (r & 7))];
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
            }
            Policy::TileDone(p, ctx, mb, nb, ew, lane);
            acc ^= 1;
            if (acc == 0) accPhase ^= 1;
        }
    }
    __syncthreads();
    if (warp == 2) { TcFenceAfter(); TmemDealloc(tmemBase, kTmemCols); }
    Policy::PostPhase(p, ctx, cta, ctas, abortWord);
    if (threadIdx.x == 0 && *abortWord != 0 && p.errorWord) *p.errorWord = 1;
    Policy::Exit(p, ctx);
}

}  // namespace mc2
}  // namespace hccl
