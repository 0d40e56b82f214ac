// Block-scaled (MXFP8) GEMM on CTA pairs: tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale, M = 256 per pair.
//
// The one-CTA block-scaled kernel (gemm_sm100_mx.cuh) is bound by shared-memory traffic the way the one-CTA bf16 kernel
// is: every stage brings 16 KB of A and 32 KB of B into one SM. Here, as in gemm_sm100_2cta.cuh, each CTA of a pair
// loads its own 128 rows of A and HALF of the B tile, and the leader's MMA thread issues instructions that read both
// CTAs' shared memory and accumulate into both CTAs' tensor memory.
//
// What block scaling adds to the pair skeleton:
//   * scale atoms (512 bytes per 128 rows x 128 K) arrive by TMA like the operands, through tensor maps over the scale
//     arrays ([atoms][128 x u32], no swizzle), because the copies of BOTH CTAs have to complete on the LEADER's barrier
//     and only the tiled form (cp.async.bulk.tensor ... .cta_group::2) may signal a barrier of the peer CTA;
//   * each CTA stages the atom of ITS rows of A and the atoms of ALL rows of the B tile (its tensor core applies B's
//     scales to all columns of its 128 x BN half of the accumulator): 0.5 KB + 1 KB per stage and CTA;
//   * the leader copies them into tensor memory of both CTAs with tcgen05.cp.cta_group::2 (same shared-memory offset,
//     same columns in both) before the four K = 32 instructions of the stage.
// Tensor memory: BN = 256 leaves room for one accumulator beside the scale columns, BN = 192 for two (a 192-wide tile
// starts at row 0 or 64 of a scale atom of B; see gemm_sm100_mx.cuh).
// No TMA multicast anywhere. Policy hooks as in the other skeletons; the scale atoms of A come from Policy::SelectSfAMap.
#pragma once
#include "gemm_sm100_2cta.cuh"
#include "gemm_sm100_mx.cuh"

namespace hccl {
namespace mc2 {

namespace cg2 {
__device__ __forceinline__ void UmmaMxf8Pair(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t sfaTmem, uint32_t sfbTmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(dTmem),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(sfaTmem), "r"(sfbTmem)
        : "memory");
}
// one scale atom from the same shared-memory offset of both CTAs into the same four columns of both CTAs' tensor memory
__device__ __forceinline__ void TmemCpSfAtomPair(uint32_t dstTmem, uint64_t smemDesc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(dstTmem), "l"(smemDesc) : "memory");
}
}  // namespace cg2

template <int BN_> struct GemmMx2CtaSmem {
    static_assert(BN_ == 192 || BN_ == 256, "tile widths of the block-scaled pair kernel");
    static constexpr int BN = BN_;
    static constexpr int kAtomsB = 2;
    static constexpr int kABytes = kBM * kMxBK;                 // 128 rows of A, 128 bytes each
    static constexpr int kBBytes = (BN / 2) * kMxBK;            // this CTA's half of the B tile
    static constexpr int kSfBytes = (1 + kAtomsB) * kSfAtomBytes;
    static constexpr int kStages = 6;
    static constexpr int kRing = kStages * (kABytes + kBBytes);
    static constexpr int kSfOff = kRing;
    static constexpr int kStageCols = 64;
    static constexpr int kStagingOff = kSfOff + kStages * kSfBytes;
    static constexpr int kStagingBytes = kBM * kStageCols * 2;
    static constexpr int kBarOff = kStagingOff + kStagingBytes;
    static constexpr int kTotal = kBarOff + 256;
    static constexpr int kAccs = BN <= 192 ? 2 : 1;
    static constexpr int kSfCols = 4 + 4 * kAtomsB;
    static constexpr int kSfColBase = kAccs * BN <= 256 ? 256 : 384;
    static_assert(kSfColBase + kStages * kSfCols <= 512, "tensor memory layout");
    static_assert(kTotal + 1024 <= 232448, "shared memory per CTA");
    static_assert(kBBytes % 1024 == 0, "B half is a whole number of swizzle atoms");
};

template <class Policy, int BN_ = 256>
__global__ void __launch_bounds__(kGemmThreads, 1) GemmKernelMx2Cta(const __grid_constant__ GemmParams p)
{
    using S = GemmMx2CtaSmem<BN_>;
    constexpr int BN = S::BN, STAGES = S::kStages, NACC = S::kAccs;
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
    const uint32_t rankInPair = cg2::CtaRankInCluster();
    const bool leader = rankInPair == 0;
    const uint32_t pair = (blockIdx.x - commCtas) >> 1, pairs = (gridDim.x - commCtas) >> 1;

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
    const uint32_t mPairs = (mBlocks + 1) / 2;
    const uint32_t numTiles = mPairs * nBlocks;
    const uint32_t kIters = p.K / kMxBK;                       // the host rejects K % 128 != 0

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { MbarInit(&tmemFull[s], 1); MbarInit(&tmemEmpty[s], 256); }
        *abortWord = 0;
        MbarInitFence();
    }
    if (warp == 2) { cg2::TmemAlloc2(tmemPtr, kTmemCols); cg2::TmemRelinquish2(); }
    TcFenceBefore();
    cg2::ClusterSync();
    TcFenceAfter();
    const uint32_t tmemBase = *tmemPtr;

    if (warp == 0) {
        if (ElectOne()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = pair; t < numTiles && ok; t += pairs) {
                uint32_t mb2, nb;
                Policy::TileCoordPairs(p, ctx, t, mPairs, nBlocks, &mb2, &nb);
                const uint32_t mb = mb2 * 2 + rankInPair;
                const bool valid = mb < mBlocks;
                const CUtensorMap *ta = &p.tmapA, *tsf = &p.tmapSfA;
                int32_t rowA = (int32_t)(mBlocks * kBM);                     // past the end: the TMA load fills zeros
                int32_t sfRowA = 0;                                          // rows past M: any finite scales do (their operands are zero)
                if (valid) {
                    ok = Policy::WaitRowsReady(p, ctx, mb, abortWord);
                    Policy::SelectA(p, ctx, mb, &ta, &rowA);
                    Policy::SelectSfAMap(p, ctx, mb, &tsf, &sfRowA);
                }
                int32_t sfRowB[S::kAtomsB];
#pragma unroll
                for (int j = 0; j < S::kAtomsB; ++j) {
                    uint32_t atom = (nb * BN) / 128 + j;
                    if (atom >= p.sfAtomsB) atom = p.sfAtomsB - 1;
                    sfRowB[j] = (int32_t)(atom * kIters);
                }
                for (uint32_t kb = 0; kb < kIters && ok; ++kb) {
                    ok = MbarWaitHint(&empty[stage], phase ^ 1, abortWord, p.waitHintNs);
                    if (!ok) break;
                    const uint32_t fullLeader = cg2::MapToCta(SmemAddr(&full[stage]), 0);
                    if (leader) MbarExpectTx(&full[stage], 2 * (S::kABytes + S::kBBytes + S::kSfBytes));
                    cg2::TmaLoad2DPair(sA + stage * S::kABytes, ta, fullLeader, (int32_t)(kb * kMxBK), rowA);
                    cg2::TmaLoad2DPair(sB + stage * S::kBBytes, &p.tmapB, fullLeader, (int32_t)(kb * kMxBK), (int32_t)(nb * BN + rankInPair * (BN / 2)));
                    uint8_t *sf = sSF + stage * S::kSfBytes;
                    cg2::TmaLoad2DPair(sf, tsf, fullLeader, 0, sfRowA + (int32_t)kb);
#pragma unroll
                    for (int j = 0; j < S::kAtomsB; ++j) cg2::TmaLoad2DPair(sf + (1 + j) * kSfAtomBytes, &p.tmapSfB, fullLeader, 0, sfRowB[j] + (int32_t)kb);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (leader && ElectOne()) {
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t t = pair; t < numTiles && ok; t += pairs) {
                uint32_t mb2, nb;
                Policy::TileCoordPairs(p, ctx, t, mPairs, nBlocks, &mb2, &nb);
                const uint32_t sfbCol = 4 + ((nb * BN) % 128) / 32;
                ok = MbarWaitHint(&tmemEmpty[acc], accPhase ^ 1, abortWord, p.waitHintNs);
                if (!ok) break;
                TcFenceAfter();
                const uint32_t dTmem = tmemBase + acc * BN;
                for (uint32_t kb = 0; kb < kIters; ++kb) {
                    ok = MbarWaitHint(&full[stage], phase, abortWord, p.waitHintNs);
                    if (!ok) break;
                    TcFenceAfter();
                    const uint32_t sfCol = tmemBase + S::kSfColBase + stage * S::kSfCols;
                    const uint32_t sfSmem = SmemAddr(sSF + stage * S::kSfBytes);
                    cg2::TmemCpSfAtomPair(sfCol, MakeSfSmemDesc(sfSmem));
#pragma unroll
                    for (int j = 0; j < S::kAtomsB; ++j) cg2::TmemCpSfAtomPair(sfCol + 4 + 4 * j, MakeSfSmemDesc(sfSmem + (1 + j) * kSfAtomBytes));
                    uint64_t aDesc = MakeSmemDescSw128(SmemAddr(sA + stage * S::kABytes));
                    uint64_t bDesc = MakeSmemDescSw128(SmemAddr(sB + stage * S::kBBytes));
#pragma unroll
                    for (uint32_t k = 0; k < kMxBK / 32; ++k)
                        cg2::UmmaMxf8Pair(dTmem, AdvanceDescK(aDesc, k * 32), AdvanceDescK(bDesc, k * 32), MakeInstrDescMx(2 * kBM, BN, k), sfCol, sfCol + sfbCol,
                                          (kb | k) != 0 ? 1u : 0u);
                    cg2::UmmaCommitPair(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                cg2::UmmaCommitPair(&tmemFull[acc]);
                if (++acc == NACC) { acc = 0; accPhase ^= 1; }
            }
        }
    } else if (warp >= 4) {
        const uint32_t ew = warp - 4;
        uint32_t acc = 0, accPhase = 0;
        bool ok = true;
        const uint32_t emptyLeader0 = cg2::MapToCta(SmemAddr(&tmemEmpty[0]), 0), emptyLeader1 = cg2::MapToCta(SmemAddr(&tmemEmpty[1]), 0);
        for (uint32_t t = pair; t < numTiles && ok; t += pairs) {
            uint32_t mb2, nb;
            Policy::TileCoordPairs(p, ctx, t, mPairs, nBlocks, &mb2, &nb);
            const uint32_t mb = mb2 * 2 + rankInPair;
            const bool valid = mb < mBlocks;
            ok = MbarWaitHint(&tmemFull[acc], accPhase, abortWord, p.waitHintNs, p.epiSleepNs);
            if (!ok) break;
            TcFenceAfter();
            const uint32_t rowInTile = ew * 32 + lane;
            const uint32_t row = mb * kBM + rowInTile;
            constexpr uint32_t SC = S::kStageCols, CH = SC / 8, kSwz = (CH - 1) & 7;
            uint4 *stg = (uint4 *)(smem + S::kStagingOff);
            const uint32_t et = threadIdx.x - 128;
            if (valid && !Policy::EpilogueGate(p, ctx, mb, abortWord)) { ok = false; break; }
#pragma unroll 1
            for (uint32_t pass = 0; pass < BN / SC; ++pass) {
#pragma unroll 1
                for (uint32_t c = 0; c < SC / 32; ++c) {
                    uint32_t v[32];
                    TmemLd32x32(tmemBase + ((ew * 32) << 16) + acc * BN + pass * SC + c * 32, v);
                    TmemLdWait();
                    if (valid) {
                        if (Policy::UseDirect(p)) {
                            Policy::Store(p, ctx, row, nb * BN + pass * SC + c * 32, v);
                            continue;
                        }
                        Policy::Combine(p, ctx, mb, row, nb * BN + pass * SC + c * 32, v);
                    }
#pragma unroll
                    for (uint32_t q = 0; q < 4; ++q) {
                        uint4 o;
                        __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
                        __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
                        __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
                        o.x = *(uint32_t *)&t0; o.y = *(uint32_t *)&t1; o.z = *(uint32_t *)&t2; o.w = *(uint32_t *)&t3;
                        stg[rowInTile * CH + ((c * 4 + q) ^ (rowInTile & kSwz))] = o;
                    }
                }
                if (pass + 1 == BN / SC) {                               // accumulator fully read: hand it back to the leader's MMA thread
                    TcFenceBefore();
                    cg2::MbarArriveRemote(acc ? emptyLeader1 : emptyLeader0);
                }
                if (Policy::UseDirect(p)) continue;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (valid) {
#pragma unroll 4
                    for (uint32_t i = et; i < (uint32_t)kBM * CH; i += 128) {
                        const uint32_t r = i / CH, ch = i % CH;
                        __nv_bfloat16 *dst = Policy::RowDst(p, ctx, mb * kBM + r, nb * BN + pass * SC + ch * 8);
                        if (dst && HCCL_RANGE_OK(dst, 16)) *(uint4 *)dst = stg[r * CH + (ch ^ (r & kSwz))];
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (valid) Policy::TileDone(p, ctx, mb, nb, ew, lane);
            if (++acc == NACC) { acc = 0; accPhase ^= 1; }
        }
    }
    // A CTA must not leave while its peer can still reach its shared memory, barriers or tensor memory.
    TcFenceBefore();
    cg2::ClusterSync();
    if (warp == 2) { TcFenceAfter(); cg2::TmemDealloc2(tmemBase, kTmemCols); }
    Policy::PostPhase(p, ctx, blockIdx.x - commCtas, gridDim.x - commCtas, abortWord);
    if (threadIdx.x == 0 && *abortWord != 0 && p.errorWord) *p.errorWord = 1;
    Policy::Exit(p, ctx);
}

}  // namespace mc2
}  // namespace hccl
