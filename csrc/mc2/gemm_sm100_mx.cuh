// Block-scaled fp8 (MXFP8) variant of the persistent tcgen05 GEMM:  C[M,N] = dequant(A)[M,K] * dequant(B)[N,K]^T with
// e4m3 operands (K-major, one byte per element) and one e8m0 scale per 1 x 32 block of K for every row of A and of B
// (the OCP microscaling format), fp32 accumulation in tensor memory, bf16 or fp32 out. The scales are applied by the
// tensor core itself (tcgen05.mma.kind::mxf8f6f4.block_scale): nothing is dequantised in registers.
//
// Same roles and the same Policy hooks as the bf16 skeleton (gemm_sm100.cuh), so the fused AllGather / ReduceScatter /
// AllReduce policies run on it unchanged. What differs:
//   * one shared-memory stage holds K = 128 elements (128 bytes per row: the same TMA boxes and 128-byte swizzle as 64
//     bf16), consumed by four K = 32 instructions;
//   * the producer also fetches the scale atoms of the stage with untiled bulk copies: 512 bytes for the 128 rows of A
//     and 512 bytes per 128 rows of B, laid out so that row r, K block k sits at (r % 32) * 16 + (r / 32) * 4 + k;
//   * before the MMAs of a stage the MMA thread copies those atoms into tensor memory (tcgen05.cp 32x128b.warpx4: 4
//     columns per atom, replicated over the four lane quarters); the four instructions pick their scale byte through
//     the scale-factor ids of the instruction descriptor;
//   * tensor memory: 256-wide tiles leave room for ONE accumulator next to the scale columns (the epilogue then does not
//     overlap the next main loop); 192- and 128-wide tiles keep two. A 192-wide tile starts at row 0 or row 64 of a scale
//     atom of B: the producer fetches the two atoms it touches and the instructions address the scale columns 0 or 2
//     columns in.
// Scale arrays are [ceil(rows / 128)][K / 128][512 bytes] (K a multiple of 128); a quantiser that writes this layout is
// in mx_quant.cu. HCCL has no counterpart (reference: include/hccl_mc2.h:25-82 only passes dtypes to external kernels).
#pragma once
#include "gemm_sm100.cuh"

namespace hccl {
namespace mc2 {

constexpr int kMxBK = 128;           // fp8 elements per stage row = 128 bytes = one swizzle row
constexpr int kSfAtomBytes = 512;
constexpr uint32_t kMxDefaultTileN = 256;     // tile width of the fused block-scaled operators unless HCCL_MX_TILE_N says otherwise

template <int BN> struct GemmMxSmem {
    static_assert(BN == 128 || BN == 192 || BN == 256, "B tiles start on a 64-row boundary of the 128-row scale atoms");
    static constexpr int kAtomsB = (BN + 127) / 128;                 // a 192-wide tile starts at row 0 or 64 of an atom: two atoms either way
    static constexpr int kABytes = kBM * kMxBK;
    static constexpr int kBBytes = BN * kMxBK;
    static constexpr int kSfBytes = (1 + kAtomsB) * kSfAtomBytes;
    static constexpr int kStages = BN >= 256 ? 4 : BN >= 192 ? 5 : 6;
    static constexpr int kRing = kStages * (kABytes + kBBytes);
    static constexpr int kSfOff = kRing;
    static constexpr int kStageCols = 64;
    static constexpr int kStagingOff = kSfOff + kStages * kSfBytes;
    static constexpr int kStagingBytes = kBM * kStageCols * 2;
    static constexpr int kBarOff = kStagingOff + kStagingBytes;
    static constexpr int kTotal = kBarOff + 256;
    // tensor memory columns
    static constexpr int kAccs = BN <= 192 ? 2 : 1;
    static constexpr int kSfCols = 4 + 4 * kAtomsB;                  // per stage: A atom, then B atoms
    static constexpr int kSfColBase = kAccs * BN <= 256 ? 256 : 384;
    static_assert(kAccs * BN <= kSfColBase && kSfColBase + kStages * kSfCols <= 512, "tensor memory layout");
    static_assert(kTotal + 1024 <= 232448, "shared memory per CTA");
};

template <int BN, class Policy, bool EMU>
__global__ void __launch_bounds__(kGemmThreads, 1) GemmKernelMx(const __grid_constant__ GemmParams pv, const GemmParams *emuParams)
{
    const GemmParams &p = EMU ? emuParams[blockIdx.y] : pv;
    using S = GemmMxSmem<BN>;
    constexpr int STAGES = S::kStages, NACC = S::kAccs;
    constexpr uint32_t kTmemCols = 512;
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);

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
    uint8_t *sSF = smem + S::kSfOff;
    uint64_t *full = (uint64_t *)(smem + S::kBarOff);
    uint64_t *empty = full + STAGES;
    uint64_t *tmemFull = empty + STAGES;
    uint64_t *tmemEmpty = tmemFull + 2;
    uint32_t *tmemPtr = (uint32_t *)(tmemEmpty + 2);
    volatile uint32_t *abortWord = (volatile uint32_t *)(tmemPtr + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t mBlocks = (p.M + kBM - 1) / kBM, nBlocks = (p.N + BN - 1) / BN;
    const uint32_t numTiles = mBlocks * nBlocks;
    const uint32_t kIters = p.K / kMxBK;                       // the host rejects K % 128 != 0

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
                const uint8_t *sfa = Policy::SelectSfA(p, ctx, mb);
                const uint8_t *sfb[S::kAtomsB];
#pragma unroll
                for (int j = 0; j < S::kAtomsB; ++j) {
                    uint32_t atom = (nb * BN) / 128 + j;
                    if (atom >= p.sfAtomsB) atom = p.sfAtomsB - 1;            // rows past N: any finite scales do (their operands are zero)
                    sfb[j] = p.sfB + (uint64_t)atom * kIters * kSfAtomBytes;
                }
                for (uint32_t kb = 0; kb < kIters && ok; ++kb) {
                    ok = MbarWaitRelaxed(&empty[stage], phase ^ 1, abortWord, p.waitSleepNs);
                    if (!ok) break;
                    MbarExpectTx(&full[stage], S::kABytes + S::kBBytes + S::kSfBytes);
                    TmaLoad2D(sA + stage * S::kABytes, ta, &full[stage], (int32_t)(kb * kMxBK), rowA);
                    TmaLoad2D(sB + stage * S::kBBytes, &p.tmapB, &full[stage], (int32_t)(kb * kMxBK), (int32_t)(nb * BN));
                    uint8_t *sf = sSF + stage * S::kSfBytes;
                    BulkLoadG2S(sf, sfa + (uint64_t)kb * kSfAtomBytes, kSfAtomBytes, &full[stage]);
#pragma unroll
                    for (int j = 0; j < S::kAtomsB; ++j)
                        BulkLoadG2S(sf + (1 + j) * kSfAtomBytes, sfb[j] + (uint64_t)kb * kSfAtomBytes, kSfAtomBytes, &full[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (ElectOne()) {
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t t = cta; t < numTiles && ok; t += ctas) {
                uint32_t mb, nb;
                Policy::TileCoord(p, ctx, t, mBlocks, nBlocks, &mb, &nb);
                // scale columns of B: 32 rows per column; a tile that starts at row 64 of its first atom starts 2 columns in
                const uint32_t sfbCol = 4 + ((nb * BN) % 128) / 32;
                ok = MbarWait(&tmemEmpty[acc], accPhase ^ 1, abortWord);
                if (!ok) break;
                TcFenceAfter();
                const uint32_t dTmem = tmemBase + acc * BN;
                for (uint32_t kb = 0; kb < kIters; ++kb) {
                    ok = MbarWait(&full[stage], phase, abortWord);
                    if (!ok) break;
                    TcFenceAfter();
                    const uint32_t sfCol = tmemBase + S::kSfColBase + stage * S::kSfCols;
                    const uint32_t sfSmem = SmemAddr(sSF + stage * S::kSfBytes);
                    TmemCpSfAtom(sfCol, MakeSfSmemDesc(sfSmem));
#pragma unroll
                    for (int j = 0; j < S::kAtomsB; ++j) TmemCpSfAtom(sfCol + 4 + 4 * j, MakeSfSmemDesc(sfSmem + (1 + j) * kSfAtomBytes));
                    uint64_t aDesc = MakeSmemDescSw128(SmemAddr(sA + stage * S::kABytes));
                    uint64_t bDesc = MakeSmemDescSw128(SmemAddr(sB + stage * S::kBBytes));
#pragma unroll
                    for (uint32_t k = 0; k < kMxBK / 32; ++k)
                        UmmaMxf8(dTmem, AdvanceDescK(aDesc, k * 32), AdvanceDescK(bDesc, k * 32), MakeInstrDescMx(kBM, BN, k), sfCol, sfCol + sfbCol,
                                 (kb | k) != 0 ? 1u : 0u);
                    UmmaCommit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                UmmaCommit(&tmemFull[acc]);
                if (++acc == NACC) { acc = 0; accPhase ^= 1; }
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
                constexpr uint32_t SC = S::kStageCols, CH = SC / 8;
                uint4 *stg = (uint4 *)(smem + S::kStagingOff);
                const uint32_t et = threadIdx.x - 128;
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
            if (++acc == NACC) { acc = 0; accPhase ^= 1; }
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
