// Policies that turn the tcgen05 GEMM skeleton into the three fused matmul + collective operators.
//
//   AgmmPolicy   AllGather + matmul: leading "comm" CTAs push the local activation shard to every peer's gather buffer
//                with bulk copies through shared memory (one counter bump per 128-row block); GEMM CTAs start with the
//                local rows and take the peers' row blocks in arrival order, gating only the TMA producer.
//   MmrsPolicy   matmul + ReduceScatter: tiles destined to other ranks are computed first and their bf16 partials are
//                stored straight into the owner's slot; after its last tile every CTA reduces a share of the rows this
//                rank owns, in rank order with fp32 accumulation.
//   MmarPolicy   matmul + AllReduce for decode-sized M: partial tiles go to the column owner, owners reduce and write the
//                result into every rank's result window, each rank copies its window to the user buffer.
#pragma once
#include "fused_common.cuh"

namespace hccl {
namespace mc2 {

// =============================================================================================== AllGather + matmul
struct AgmmPolicy {
    using Ctx = FusedCtx;
    // u64: 0 gatherOff (half 0), 1 gatherBytes per half, 2 aLocal, 3 scale window (half 0) and 5 local scale atoms (block-scaled operands)
    // u32: 0 mLocal, 1 commCtas, 2 blocksPerRank, 3 pieces per 128-row block pushed by spare warps (0 = comm CTAs push whole blocks)
    __device__ static void Init(const GemmParams &p, Ctx &x) { FusedInit(p, x); }
    __device__ static uint32_t CommCtas(const GemmParams &p) { return p.u32[1]; }

    __device__ static void CommRole(const GemmParams &p, Ctx &x, uint8_t *smem)
    {
        constexpr uint32_t SLOTS = 8, PIECE = 16384;
        uint64_t *full = (uint64_t *)(smem + SLOTS * PIECE);
        uint64_t *empty = full + SLOTS;
        volatile uint32_t *abortWord = (volatile uint32_t *)(empty + SLOTS);
        if (threadIdx.x == 0) {
            for (uint32_t s = 0; s < SLOTS; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
            *abortWord = 0;
            MbarInitFence();
        }
        __syncthreads();
        const uint32_t bpr = p.u32[2], n = (uint32_t)x.n, C = p.u32[1];
        // Every (peer, 128-row block) item moves up to two segments: the rows themselves and, for block-scaled operands,
        // the block's scale atoms (u64[3] = scale window of half 0 inside the heap, u64[5] = local scale array).
        const uint32_t eb = p.elemBytes ? p.elemBytes : 2;
        const uint64_t segBytes[2] = {(uint64_t)kBM * p.K * eb, p.u64[5] ? (uint64_t)(p.K / 128) * 512 : 0};
        const char *segSrc[2] = {(const char *)p.u64[2], (const char *)p.u64[5]};
        const uint64_t segDstBase[2] = {p.u64[0] + (uint64_t)x.half * p.u64[1], p.u64[3] + (uint64_t)x.half * p.u64[1]};
        const uint32_t nseg = segBytes[1] ? 2 : 1;
        const uint32_t items = (n - 1) * bpr;
        const uint32_t warp = threadIdx.x >> 5;
        if (warp == 0 && ElectOne()) {            // loader: local shard -> shared memory ring
            uint32_t j = 0;
            for (uint32_t it = blockIdx.x; it < items; it += C) {
                uint32_t blk = it % bpr;
                for (uint32_t g = 0; g < nseg; ++g) {
                    const char *src = segSrc[g] + (uint64_t)blk * segBytes[g];
                    const uint32_t pieces = (uint32_t)((segBytes[g] + PIECE - 1) / PIECE);
                    for (uint32_t q = 0; q < pieces; ++q, ++j) {
                        uint32_t s = j % SLOTS, ph = (j / SLOTS) & 1;
                        if (!MbarWait(&empty[s], ph ^ 1, abortWord)) return;
                        uint32_t bytes = (uint32_t)(segBytes[g] - (uint64_t)q * PIECE < PIECE ? segBytes[g] - (uint64_t)q * PIECE : PIECE);
                        MbarExpectTx(&full[s], bytes);
                        BulkLoad(smem + s * PIECE, src + (uint64_t)q * PIECE, bytes, &full[s]);
                    }
                }
            }
        } else if (warp == 1 && ElectOne()) {     // storer: ring -> the peer's gather buffer, then bump its counter
            uint32_t j = 0, rel = 0;              // pieces stored / ring slots handed back to the loader
            for (uint32_t it = blockIdx.x; it < items; it += C) {
                uint32_t d = it / bpr + 1, blk = it % bpr;
                uint32_t peer = ((uint32_t)x.rank + d) % n;
                for (uint32_t g = 0; g < nseg; ++g) {
                    char *dst = x.c->heap[peer] + segDstBase[g] + ((uint64_t)x.rank * bpr + blk) * segBytes[g];
                    const uint32_t pieces = (uint32_t)((segBytes[g] + PIECE - 1) / PIECE);
                    for (uint32_t q = 0; q < pieces; ++q, ++j) {
                        uint32_t s = j % SLOTS, ph = (j / SLOTS) & 1;
                        if (!MbarWait(&full[s], ph, abortWord)) return;
                        uint32_t bytes = (uint32_t)(segBytes[g] - (uint64_t)q * PIECE < PIECE ? segBytes[g] - (uint64_t)q * PIECE : PIECE);
                        BulkStore(dst + (uint64_t)q * PIECE, smem + s * PIECE, bytes);
                        TmaStoreCommit();
                        BulkWaitRead<1>();             // every piece before this one has left shared memory
                        for (; rel < j; ++rel) MbarArrive(&empty[rel % SLOTS]);
                    }
                }
                TmaStoreWaitAll();                 // every byte of this block is written at the peer
                for (; rel < j; ++rel) MbarArrive(&empty[rel % SLOTS]);
                FenceProxyAsyncGlobal();
                __threadfence_system();
                RemoteAddRelease(&FlagsOf(x.c->heap[peer])->mc2Ready[x.half][x.rank][blk], 1u);
            }
        }
    }

    __device__ static void TileCoord(const GemmParams &p, const Ctx &x, uint32_t t, uint32_t, uint32_t nBlocks, uint32_t *mb, uint32_t *nb)
    {
        const uint32_t bpr = p.u32[2], perSrc = bpr * nBlocks;
        uint32_t d = t / perSrc, rem = t % perSrc;
        uint32_t src = ((uint32_t)x.rank + (uint32_t)x.n - d % (uint32_t)x.n) % (uint32_t)x.n;
        uint32_t blk;
        SegmentTile(rem, bpr, nBlocks, &blk, nb);
        *mb = src * bpr + blk;
    }
    // CTA-pair kernel without communication CTAs: warps 2 and 3 of every GEMM CTA push pieces of the local shard to the
    // peers with plain 16-byte loads / peer stores, nearest consumer first, one counter bump per piece.
    __device__ static void SpareWarps(const GemmParams &p, Ctx &x, uint32_t which, uint32_t cta, uint32_t ctas, uint32_t lane, volatile uint32_t *)
    {
        const uint32_t P = p.u32[3];
        if (P == 0) return;
        const uint32_t bpr = p.u32[2], n = (uint32_t)x.n;
        const uint32_t items = (n - 1) * bpr * P, worker = cta * 2 + which, workers = ctas * 2;
        const uint64_t rowBytes = (uint64_t)p.K * (p.elemBytes ? p.elemBytes : 2), pieceRows = kBM / P, pieceBytes = pieceRows * rowBytes;
        const char *aLocal = (const char *)p.u64[2];
        const uint64_t gatherBase = p.u64[0] + (uint64_t)x.half * p.u64[1];
        for (uint32_t it = worker; it < items; it += workers) {
            const uint32_t d = it / (bpr * P) + 1, rem = it % (bpr * P), blk = rem / P, piece = rem % P;
            const uint32_t peer = ((uint32_t)x.rank + d) % n;
            const uint64_t rowOff = ((uint64_t)blk * kBM + (uint64_t)piece * pieceRows) * rowBytes;
            const uint4 *src = (const uint4 *)(aLocal + rowOff);
            uint4 *dst = (uint4 *)(x.c->heap[peer] + gatherBase + (uint64_t)x.rank * p.u32[0] * rowBytes + rowOff);
            const uint64_t nvec = pieceBytes >> 4;
            constexpr int U = 8;
            uint64_t i = lane;
            for (; i + 32ull * (U - 1) < nvec; i += 32ull * U) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = src[i + 32ull * u];
#pragma unroll
                for (int u = 0; u < U; ++u) dst[i + 32ull * u] = v[u];
            }
            for (; i < nvec; i += 32) dst[i] = src[i];
            __syncwarp();
            if (lane == 0) {
                __threadfence_system();
                RemoteAddRelease(&FlagsOf(x.c->heap[peer])->mc2Ready[x.half][x.rank][blk], 1u);
            }
        }
    }
    // CTA-pair kernel (blocks per rank even): the same source order over pairs of row blocks
    __device__ static void TileCoordPairs(const GemmParams &p, const Ctx &x, uint32_t t, uint32_t, uint32_t nBlocks, uint32_t *mb2, uint32_t *nb)
    {
        const uint32_t ppr = p.u32[2] / 2, perSrc = ppr * nBlocks;
        uint32_t d = t / perSrc, rem = t % perSrc;
        uint32_t src = ((uint32_t)x.rank + (uint32_t)x.n - d % (uint32_t)x.n) % (uint32_t)x.n;
        uint32_t blk2;
        SegmentTile(rem, ppr, nBlocks, &blk2, nb, 8);
        *mb2 = src * ppr + blk2;
    }
    __device__ static bool WaitRowsReady(const GemmParams &p, const Ctx &x, uint32_t mb, volatile uint32_t *abortWord)
    {
        const uint32_t bpr = p.u32[2], src = mb / bpr, blk = mb % bpr;
        if ((int)src == x.rank) return true;
        Ctx &xm = const_cast<Ctx &>(x);
        bool ok = WaitCounterGe(xm, &x.flags->mc2Ready[x.half][src][blk], p.u32[3] ? p.u32[3] : 1u, src, 31, abortWord);
        asm volatile("fence.proxy.async;" ::: "memory");   // peer's generic/async writes -> this CTA's TMA reads
        return ok;
    }
    __device__ static void SelectA(const GemmParams &p, const Ctx &x, uint32_t mb, const CUtensorMap **tm, int32_t *row)
    {
        const uint32_t bpr = p.u32[2], src = mb / bpr, blk = mb % bpr;
        if ((int)src == x.rank) { *tm = &p.tmapALocal; *row = (int32_t)(blk * kBM); }
        else { *tm = x.half ? &p.tmapA1 : &p.tmapA; *row = (int32_t)(mb * kBM); }
    }
    // block-scaled operands: scale atoms of row block mb -- the local array for the own rows, the gathered window otherwise
    __device__ static const uint8_t *SelectSfA(const GemmParams &p, const Ctx &x, uint32_t mb)
    {
        const uint32_t bpr = p.u32[2], src = mb / bpr, blk = mb % bpr;
        const uint64_t blockSf = (uint64_t)(p.K / 128) * 512;
        if ((int)src == x.rank) return (const uint8_t *)p.u64[5] + (uint64_t)blk * blockSf;
        return (const uint8_t *)x.heap + p.u64[3] + (uint64_t)x.half * p.u64[1] + (uint64_t)mb * blockSf;
    }
    // the same through tensor maps (CTA-pair kernel): the local scale array, or the gathered window of this parity half
    __device__ static void SelectSfAMap(const GemmParams &p, const Ctx &x, uint32_t mb, const CUtensorMap **tm, int32_t *atomRow)
    {
        const uint32_t bpr = p.u32[2], src = mb / bpr, blk = mb % bpr;
        if ((int)src == x.rank) { *tm = &p.tmapSfALocal; *atomRow = (int32_t)(blk * (p.K / 128)); }
        else { *tm = x.half ? &p.tmapSfA1 : &p.tmapSfA; *atomRow = (int32_t)(mb * (p.K / 128)); }
    }
    __device__ static bool UseDirect(const GemmParams &) { return false; }
    __device__ static void Store(const GemmParams &, const Ctx &, uint32_t, uint32_t, const uint32_t (&)[32]) {}
    __device__ static __nv_bfloat16 *RowDst(const GemmParams &p, const Ctx &, uint32_t row, uint32_t col)
    {
        return (row < p.M && col < p.N) ? (__nv_bfloat16 *)p.C + (size_t)row * p.ldc + col : nullptr;
    }
    __device__ static bool EpilogueGate(const GemmParams &, Ctx &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void Combine(const GemmParams &, const Ctx &, uint32_t, uint32_t, uint32_t, uint32_t (&)[32]) {}
    __device__ static void TileDone(const GemmParams &, const Ctx &, uint32_t, uint32_t, uint32_t, uint32_t) {}
    __device__ static void PostPhase(const GemmParams &, Ctx &, uint32_t, uint32_t, volatile uint32_t *) {}
    __device__ static void Exit(const GemmParams &, Ctx &x) { FusedExit(x); }
};

// Stores 32 fp32 accumulators of one row as bf16 (64 bytes) at `dst` (16-byte aligned, local or peer memory).
__device__ __forceinline__ void StoreBf16x32(__nv_bfloat16 *dst, const uint32_t (&v)[32], uint32_t validCols = 32)
{
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        if ((uint32_t)j >= validCols) break;
        uint4 o;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
        __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
        __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
        __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
        o.x = *(uint32_t *)&t0; o.y = *(uint32_t *)&t1; o.z = *(uint32_t *)&t2; o.w = *(uint32_t *)&t3;
        *(uint4 *)(dst + j) = o;
    }
}

// acc[0..7] (+)= the 8 bf16 values of `raw`
__device__ __forceinline__ void AccumBf16x8(float (&acc)[8], uint4 raw, bool first)
{
    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        if (first) { acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
        else { acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
}
__device__ __forceinline__ uint4 PackBf16x8(const float (&acc)[8])
{
    uint4 o;
    __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0], acc[1]), t1 = __floats2bfloat162_rn(acc[2], acc[3]);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4], acc[5]), t3 = __floats2bfloat162_rn(acc[6], acc[7]);
    o.x = *(uint32_t *)&t0; o.y = *(uint32_t *)&t1; o.z = *(uint32_t *)&t2; o.w = *(uint32_t *)&t3;
    return o;
}

// 128 epilogue threads (warps 4..7) meet on named barrier 1
__device__ __forceinline__ void EpilogueBarrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// =============================================================================================== matmul + ReduceScatter
struct MmrsPolicy {
    using Ctx = FusedCtx;
    // u64: 0 wsOff (half 0), 1 wsBytes per half   u32: 0 mOwn (rows per rank), 1 blocksPerOwner, 2 nBlocks (N / BN)
    __device__ static void Init(const GemmParams &p, Ctx &x) { FusedInit(p, x); }
    __device__ static uint32_t CommCtas(const GemmParams &) { return 0; }
    __device__ static void CommRole(const GemmParams &, Ctx &, uint8_t *) {}
    // other owners first (rank+1, rank+2, ...), own rows last
    __device__ static void TileCoord(const GemmParams &p, const Ctx &x, uint32_t t, uint32_t, uint32_t nBlocks, uint32_t *mb, uint32_t *nb)
    {
        const uint32_t bpo = p.u32[1], perOwner = bpo * nBlocks, n = (uint32_t)x.n;
        uint32_t d = t / perOwner, rem = t % perOwner;
        uint32_t owner = ((uint32_t)x.rank + 1 + d) % n;
        uint32_t blk;
        SegmentTile(rem, bpo, nBlocks, &blk, nb);
        *mb = owner * bpo + blk;
    }
    __device__ static void SpareWarps(const GemmParams &, Ctx &, uint32_t, uint32_t, uint32_t, uint32_t, volatile uint32_t *) {}
    __device__ static void TileCoordPairs(const GemmParams &p, const Ctx &x, uint32_t t, uint32_t, uint32_t nBlocks, uint32_t *mb2, uint32_t *nb)
    {
        const uint32_t ppo = p.u32[1] / 2, perOwner = ppo * nBlocks, n = (uint32_t)x.n;
        uint32_t d = t / perOwner, rem = t % perOwner;
        uint32_t owner = ((uint32_t)x.rank + 1 + d) % n;
        uint32_t blk2;
        SegmentTile(rem, ppo, nBlocks, &blk2, nb, 8);
        *mb2 = owner * ppo + blk2;
    }
    __device__ static bool WaitRowsReady(const GemmParams &, const Ctx &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void SelectA(const GemmParams &p, const Ctx &, uint32_t mb, const CUtensorMap **tm, int32_t *row)
    {
        *tm = &p.tmapA;
        *row = (int32_t)(mb * kBM);
    }
    __device__ static const uint8_t *SelectSfA(const GemmParams &p, const Ctx &, uint32_t mb) { return p.sfA + (uint64_t)mb * (p.K / 128) * 512; }
    __device__ static void SelectSfAMap(const GemmParams &p, const Ctx &, uint32_t mb, const CUtensorMap **tm, int32_t *atomRow)
    {
        *tm = &p.tmapSfA;
        *atomRow = (int32_t)(mb * (p.K / 128));
    }
    __device__ static bool UseDirect(const GemmParams &) { return false; }
    __device__ static void Store(const GemmParams &, const Ctx &, uint32_t, uint32_t, const uint32_t (&)[32]) {}
    // Tiles of rows owned by a peer: the bf16 partial goes into slot[rank] of the owner's workspace. Tiles of the own
    // rows come last; by then the peers' partials have long arrived, so their epilogue adds them (rank order, fp32) to
    // the accumulator and writes the final result: no separate reduction pass, no round trip of the own partial.
    __device__ static __nv_bfloat16 *RowDst(const GemmParams &p, const Ctx &x, uint32_t row, uint32_t col)
    {
        if (row >= p.M || col >= p.N) return nullptr;
        const uint32_t mOwn = p.u32[0], owner = row / mOwn, r = row - owner * mOwn;
        if ((int)owner == x.rank) return (__nv_bfloat16 *)p.C + (uint64_t)r * p.ldc + col;
        char *ws = x.c->heap[owner] + p.u64[0] + (uint64_t)x.half * p.u64[1];
        return (__nv_bfloat16 *)ws + ((uint64_t)x.rank * mOwn + r) * p.N + col;
    }
    __device__ static bool EpilogueGate(const GemmParams &p, Ctx &x, uint32_t mb, volatile uint32_t *abortWord)
    {
        const uint32_t bpo = p.u32[1], owner = mb / bpo, blk = mb % bpo, nBlocks = p.u32[2];
        if ((int)owner != x.rank) return true;
        const uint32_t et = threadIdx.x - 128;
        if (et < (uint32_t)x.n && (int)et != x.rank) WaitCounterGe(x, &x.flags->mc2Ready[x.half][et][blk], nBlocks, et, 41, abortWord);
        EpilogueBarrier();
        return *abortWord == 0;
    }
    __device__ static void Combine(const GemmParams &p, const Ctx &x, uint32_t mb, uint32_t row, uint32_t col0, uint32_t (&v)[32])
    {
        const uint32_t mOwn = p.u32[0], bpo = p.u32[1];
        if ((int)(mb / bpo) != x.rank || row >= p.M || col0 >= p.N) return;
        const uint32_t r = row - (uint32_t)x.rank * mOwn, n = (uint32_t)x.n;
        const __nv_bfloat16 *ws = (const __nv_bfloat16 *)(x.heap + p.u64[0] + (uint64_t)x.half * p.u64[1]);
        const uint32_t valid = p.N - col0 < 32 ? p.N - col0 : 32;
        // Eight columns at a time: the partial rows of ALL sources are requested before any is used (one round trip to memory per
        // eight columns instead of one per source), then added in rank order with the own accumulator in its place, so the result
        // has the same bits as a source-by-source walk.
        constexpr uint32_t kSrc = 8;
        const uint64_t rowOff = (uint64_t)r * p.N + col0;
        float sum[32];
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
            if (q * 8 >= valid) {
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[q * 8 + j] = __uint_as_float(v[q * 8 + j]);
                continue;
            }
            float acc[8];
            bool first = true;
            for (uint32_t s0 = 0; s0 < n; s0 += kSrc) {
                uint4 raw[kSrc];
#pragma unroll
                for (uint32_t i = 0; i < kSrc; ++i) {
                    const uint32_t s = s0 + i;
                    if (s < n && (int)s != x.rank) raw[i] = ((const uint4 *)(ws + (uint64_t)s * mOwn * p.N + rowOff))[q];
                }
#pragma unroll
                for (uint32_t i = 0; i < kSrc; ++i) {
                    const uint32_t s = s0 + i;
                    if (s >= n) break;
                    if ((int)s == x.rank) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = first ? __uint_as_float(v[q * 8 + j]) : acc[j] + __uint_as_float(v[q * 8 + j]);
                    } else {
                        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw[i];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float2 f = __bfloat1622float2(h[j]);
                            acc[2 * j] = first ? f.x : acc[2 * j] + f.x;
                            acc[2 * j + 1] = first ? f.y : acc[2 * j + 1] + f.y;
                        }
                    }
                    first = false;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[q * 8 + j] = acc[j];
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(sum[j]);
    }
    __device__ static void TileDone(const GemmParams &p, const Ctx &x, uint32_t mb, uint32_t, uint32_t ew, uint32_t lane)
    {
        const uint32_t bpo = p.u32[1], owner = mb / bpo, blk = mb % bpo;
        if ((int)owner == x.rank) return;
        if (ew == 0 && lane == 0) {     // the write-out ended with a barrier of the 128 epilogue threads
            __threadfence_system();
            RemoteAddRelease(&FlagsOf(x.c->heap[owner])->mc2Ready[x.half][x.rank][blk], 1u);
        }
    }
    __device__ static void PostPhase(const GemmParams &, Ctx &, uint32_t, uint32_t, volatile uint32_t *) {}
    __device__ static void Exit(const GemmParams &, Ctx &x) { FusedExit(x); }
};

// =============================================================================================== matmul + AllReduce (decode)
struct MmarPolicy {
    using Ctx = FusedCtx;
    // u64: 0 wsOff, 1 wsBytes per half ([src][M][colsOwn] bf16), 2 resOff, 3 resBytes per half ([M][N] bf16)
    // u32: 0 colsOwn (N / ranks), 1 tilesPerOwnerRow (colsOwn / BN), 2 BN
    __device__ static void Init(const GemmParams &p, Ctx &x) { FusedInit(p, x); }
    __device__ static uint32_t CommCtas(const GemmParams &) { return 0; }
    __device__ static void CommRole(const GemmParams &, Ctx &, uint8_t *) {}
    __device__ static void TileCoord(const GemmParams &, const Ctx &x, uint32_t t, uint32_t mBlocks, uint32_t nBlocks, uint32_t *mb, uint32_t *nb)
    {
        // rotate the column blocks so that every rank starts with tiles owned by its right neighbour
        uint32_t nbRaw = t / mBlocks;
        uint32_t shift = ((uint32_t)x.rank + 1) * (nBlocks / (uint32_t)x.n);
        *nb = (nbRaw + shift) % nBlocks;
        *mb = t % mBlocks;
    }
    __device__ static bool WaitRowsReady(const GemmParams &, const Ctx &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void SelectA(const GemmParams &p, const Ctx &, uint32_t mb, const CUtensorMap **tm, int32_t *row)
    {
        *tm = &p.tmapA;
        *row = (int32_t)(mb * kBM);
    }
    __device__ static const uint8_t *SelectSfA(const GemmParams &p, const Ctx &, uint32_t mb) { return p.sfA + (uint64_t)mb * (p.K / 128) * 512; }
    __device__ static bool UseDirect(const GemmParams &) { return false; }
    __device__ static void Store(const GemmParams &, const Ctx &, uint32_t, uint32_t, const uint32_t (&)[32]) {}
    __device__ static __nv_bfloat16 *RowDst(const GemmParams &p, const Ctx &x, uint32_t row, uint32_t col)
    {
        if (row >= p.M || col >= p.N) return nullptr;
        const uint32_t colsOwn = p.u32[0], owner = col / colsOwn;
        char *ws = x.c->heap[owner] + p.u64[0] + (uint64_t)x.half * p.u64[1];
        return (__nv_bfloat16 *)ws + ((uint64_t)x.rank * p.M + row) * colsOwn + (col - owner * colsOwn);
    }
    __device__ static bool EpilogueGate(const GemmParams &, Ctx &, uint32_t, volatile uint32_t *) { return true; }
    __device__ static void Combine(const GemmParams &, const Ctx &, uint32_t, uint32_t, uint32_t, uint32_t (&)[32]) {}
    __device__ static uint32_t CounterIndex(const GemmParams &p, uint32_t mb, uint32_t nb)
    {
        return (mb * p.u32[1] + nb % p.u32[1]) & 63u;
    }
    __device__ static void TileDone(const GemmParams &p, const Ctx &x, uint32_t mb, uint32_t nb, uint32_t ew, uint32_t lane)
    {
        EpilogueBarrier();
        if (ew == 0 && lane == 0) {
            const uint32_t owner = nb / p.u32[1];
            __threadfence_system();
            RemoteAddRelease(&FlagsOf(x.c->heap[owner])->mc2Ready[x.half][x.rank][CounterIndex(p, mb, nb)], 1u);
        }
    }
    __device__ static void PostPhase(const GemmParams &p, Ctx &x, uint32_t cta, uint32_t ctas, volatile uint32_t *abortWord)
    {
        const uint32_t colsOwn = p.u32[0], tpr = p.u32[1], BN = p.u32[2], n = (uint32_t)x.n;
        const uint32_t mBlocks = (p.M + kBM - 1) / kBM;
        // reduce units: each owned tile is cut into row chunks so that there is about one unit per CTA
        uint32_t rowChunks = ctas / (mBlocks * tpr);
        rowChunks = rowChunks >= 8 ? 8 : rowChunks >= 4 ? 4 : rowChunks >= 2 ? 2 : 1;
        const uint32_t ROWS = kBM / rowChunks;
        const uint32_t units = mBlocks * tpr * rowChunks;    // reduce units this rank owns
        const char *ws = x.heap + p.u64[0] + (uint64_t)x.half * p.u64[1];
        const uint64_t resBase = p.u64[2] + (uint64_t)x.half * p.u64[3];
        // stage A: reduce the tiles this rank owns and write the result into every rank's result window
        for (uint32_t u = cta; u < units; u += ctas) {
            const uint32_t tile = u / rowChunks, rc = u % rowChunks, mb = tile / tpr, tc = tile % tpr;
            bool mine = true;
            if (threadIdx.x < n) mine = WaitCounterGe(x, &x.flags->mc2Ready[x.half][threadIdx.x][(mb * tpr + tc) & 63u], 1u, threadIdx.x, 51, abortWord);
            if (!__syncthreads_and(mine ? 1 : 0)) return;
            const uint32_t vecPerRow = BN / 8;
            for (uint32_t v = threadIdx.x; v < ROWS * vecPerRow; v += blockDim.x) {
                const uint32_t r = mb * kBM + rc * ROWS + v / vecPerRow, c = tc * BN + (v % vecPerRow) * 8;
                if (r >= p.M) continue;
                float acc[8];
                for (uint32_t s = 0; s < n; ++s) {
                    uint4 raw = *(const uint4 *)((const __nv_bfloat16 *)ws + ((uint64_t)s * p.M + r) * colsOwn + c);
                    AccumBf16x8(acc, raw, s == 0);
                }
                uint4 packed = PackBf16x8(acc);
                for (uint32_t q = 0; q < n; ++q) {
                    uint32_t dstRank = ((uint32_t)x.rank + q) % n;
                    *(uint4 *)((__nv_bfloat16 *)(x.c->heap[dstRank] + resBase) + (uint64_t)r * p.N + (uint64_t)x.rank * colsOwn + c) = packed;
                }
            }
            __syncthreads();
            if (threadIdx.x < n) {
                __threadfence_system();
                RemoteAddRelease(&FlagsOf(x.c->heap[threadIdx.x])->mc2Done[x.half][x.rank][0], 1u);
            }
        }
        // stage B: all owners have delivered -> copy the result window to the user buffer
        bool mine = true;
        if (threadIdx.x < n) mine = WaitCounterGe(x, &x.flags->mc2Done[x.half][threadIdx.x][0], units, threadIdx.x, 52, abortWord);
        if (!__syncthreads_and(mine ? 1 : 0)) return;
        dev::Part part = dev::PartOf((uint64_t)p.M * p.N * 2, ctas, cta);
        dev::BlockCopy((char *)p.C + part.off, x.heap + resBase + part.off, part.len);
    }
    __device__ static void Exit(const GemmParams &, Ctx &x) { FusedExit(x); }
};

}  // namespace mc2
}  // namespace hccl
