// Two-CTA (cta_group::2) variant of the persistent tcgen05 GEMM: a thread-block cluster of two CTAs on neighbouring SMs
// computes one 256 x 256 output tile. Each CTA loads its own 128 rows of A and HALF of the B tile (128 of the 256
// rows), the leader CTA's MMA thread issues tcgen05.mma.cta_group::2 (M = 256) which reads both CTAs' shared memory and
// accumulates into both CTAs' tensor memory (128 lanes each), and each CTA's epilogue warps drain their own half.
// Per SM and k-block this moves 32 KB instead of the 48 KB of the one-CTA 128 x 256 tile, which is what bounds the
// one-CTA kernel (its tensor pipe waits for L2).
//
// Cross-CTA signalling (no TMA multicast anywhere):
//   full[s]      lives in the LEADER: the leader's producer arms it with the bytes of both CTAs, and both CTAs' TMA loads
//                complete on it (cp.async.bulk.tensor ... .cta_group::2 with the leader's barrier address)
//   empty[s]     one per CTA, released for both by tcgen05.commit.cta_group::2 ... multicast::cluster
//   tmemFull[a]  one per CTA, same multicast commit after the last k-block of a tile
//   tmemEmpty[a] lives in the LEADER with 256 arrivals: the epilogue threads of both CTAs (the peer's arrive remotely)
// The Policy hooks are those of the one-CTA skeleton; they are called with 128-row block indices, so a fused policy
// needs no change: CTA r of the pair works on row block 2 * mb2 + r.
#pragma once
#include "gemm_sm100.cuh"

namespace hccl {
namespace mc2 {

namespace cg2 {
__device__ __forceinline__ uint32_t CtaRankInCluster()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void ClusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `smemAddr` (a shared::cta address of this CTA) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t MapToCta(uint32_t smemAddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void MbarArriveRemote(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// tiled load into THIS CTA's shared memory, completion bytes on a barrier given by its shared::cluster address
__device__ __forceinline__ void TmaLoad2DPair(void *smemDst, const CUtensorMap *m, uint32_t barClusterAddr, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     SmemAddr(smemDst)),
                 "l"(m), "r"(barClusterAddr), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void TmemAlloc2(uint32_t *smemOut, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemOut)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemDealloc2(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void UmmaF16Pair(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at the same shared-memory offset in both CTAs of the pair once the issued MMAs have completed
__device__ __forceinline__ void UmmaCommitPair(uint64_t *bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "h"(mask)
                 : "memory");
}
}  // namespace cg2

template <int BN_> struct Gemm2CtaSmemT {
    static constexpr int BN = BN_;                           // 256, or 224 when that wastes fewer tile waves
    static constexpr int kStages = 6;
    static constexpr int kABytes = kBM * kBK * 2;            // 128 rows of A
    static constexpr int kBBytes = (BN / 2) * kBK * 2;       // this CTA's half of the B tile (a multiple of the 1 KB swizzle atom)
    static constexpr int kRing = kStages * (kABytes + kBBytes);
    static constexpr int kStageCols = BN % 64 == 0 ? 64 : 32;
    static constexpr int kStagingOff = kRing;
    static constexpr int kStagingBytes = kBM * kStageCols * 2;
    static constexpr int kBarOff = kRing + kStagingBytes;
    static constexpr int kTotal = kBarOff + 256;
};
using Gemm2CtaSmem = Gemm2CtaSmemT<256>;

template <class Policy, int BN_ = 256>
__global__ void __launch_bounds__(kGemmThreads, 1) GemmKernel2Cta(const __grid_constant__ GemmParams p)
{
    using S = Gemm2CtaSmemT<BN_>;
    constexpr int BN = S::BN, STAGES = S::kStages;
    constexpr uint32_t kTmemCols = 512;                                        // two 256-column accumulators
    constexpr uint32_t kIdesc = MakeInstrDesc(FMT_BF16, FMT_BF16, 2 * kBM, BN);
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);

    typename Policy::Ctx ctx;
    Policy::Init(p, ctx);
    const uint32_t commCtas = Policy::CommCtas(p);          // an even number: whole pairs run the communication role
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
    const uint32_t kIters = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { MbarInit(&tmemFull[s], 1); MbarInit(&tmemEmpty[s], 256); }
        *abortWord = 0;
        MbarInitFence();
    }
    if (warp == 2) { cg2::TmemAlloc2(tmemPtr, kTmemCols); cg2::TmemRelinquish2(); }
    TcFenceBefore();
    cg2::ClusterSync();                     // both CTAs' barriers are initialised before anything remote touches them
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
                const CUtensorMap *ta = &p.tmapA;
                int32_t rowA = (int32_t)(mBlocks * kBM);                     // past the end: the TMA load fills zeros
                if (valid) {
                    ok = Policy::WaitRowsReady(p, ctx, mb, abortWord);
                    Policy::SelectA(p, ctx, mb, &ta, &rowA);
                }
                for (uint32_t kb = 0; kb < kIters && ok; ++kb) {
                    ok = MbarWaitHint(&empty[stage], phase ^ 1, abortWord, p.waitHintNs);
                    if (!ok) break;
                    const uint32_t fullLeader = cg2::MapToCta(SmemAddr(&full[stage]), 0);
                    if (leader) MbarExpectTx(&full[stage], 2 * (S::kABytes + S::kBBytes));
                    cg2::TmaLoad2DPair(sA + stage * S::kABytes, ta, fullLeader, (int32_t)(kb * kBK), rowA);
                    cg2::TmaLoad2DPair(sB + stage * S::kBBytes, &p.tmapB, fullLeader, (int32_t)(kb * kBK), (int32_t)(nb * BN + rankInPair * (BN / 2)));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (leader && ElectOne()) {
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t t = pair; t < numTiles && ok; t += pairs) {
                ok = MbarWaitHint(&tmemEmpty[acc], accPhase ^ 1, abortWord, p.waitHintNs);
                if (!ok) break;
                TcFenceAfter();
                const uint32_t dTmem = tmemBase + acc * BN;
                for (uint32_t kb = 0; kb < kIters; ++kb) {
                    ok = MbarWaitHint(&full[stage], phase, abortWord, p.waitHintNs);
                    if (!ok) break;
                    TcFenceAfter();
                    uint64_t aDesc = MakeSmemDescSw128(SmemAddr(sA + stage * S::kABytes));
                    uint64_t bDesc = MakeSmemDescSw128(SmemAddr(sB + stage * S::kBBytes));
#pragma unroll
                    for (uint32_t k = 0; k < kBK / 16; ++k)
                        cg2::UmmaF16Pair(dTmem, AdvanceDescK(aDesc, k * 32), AdvanceDescK(bDesc, k * 32), kIdesc, (kb | k) != 0 ? 1u : 0u);
                    cg2::UmmaCommitPair(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                cg2::UmmaCommitPair(&tmemFull[acc]);
                acc ^= 1;
                if (acc == 0) accPhase ^= 1;
            }
        }
    } else if (warp == 2 || warp == 3) {
        // spare warps: a fused policy may move data with them (AllGatherMatmul pushes the local shard to the peers)
        Policy::SpareWarps(p, ctx, warp - 2, blockIdx.x - commCtas, gridDim.x - commCtas, lane, abortWord);
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
            constexpr uint32_t SC = S::kStageCols, CH = SC / 8, kSwz = (CH - 1) & 7;   // bank-conflict swizzle within a staged row
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
            acc ^= 1;
            if (acc == 0) accPhase ^= 1;
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
