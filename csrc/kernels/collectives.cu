// Collective kernels of the SM and NVLS engines (sm_100a). Each operator chunk is ONE launch: data movement over
// NVLink by plain peer loads/stores (or multimem.* through the NVSwitch multicast mapping), reduction in registers
// in rank order, synchronisation by epoch flags in the symmetric heap with bounded waits.
//
// Shapes follow HCCL's vector-core kernel family (reference: src/ops/all_reduce/template/aiv/kernel/
// aiv_all_reduce_mesh_1d_oneshot.h:17-120 and ..._twoshot.h:16-349, all_gather/.../aiv_all_gather_mesh_1d.h:17-237,
// reduce_scatter/.../aiv_reduce_scatter_mesh_1d.h:16-93, all_to_all_v/.../aiv_all_to_all_v_mesh_1D.h:16-271,
// broadcast/.../aiv_broadcast_mesh_1d.h, reduce/.../aiv_reduce_mesh_1d.h, scatter/.../aiv_scatter_mesh_1d.h,
// send/recv .../aiv_send_mesh_1D.h:42-56) but are laid out for NVSwitch: every CTA ("channel") owns the same byte
// range on every rank, so ranks synchronise per channel and never grid-wide, and no kernel ends with a barrier:
// the two CCL halves alternate per operator (device-resident parity), and every operator contains at least one
// all-peer synchronisation, so a rank entering operator k+2 knows every peer has left operator k.
//
// EMU = true: all ranks live on one GPU and blockIdx.y is the rank; launched cooperatively so that the CTAs that
// wait for each other are co-resident. Used to test the protocols on a single device.
#include <cooperative_groups.h>
#include "coll_args.h"
#include "primitives.cuh"

namespace hccl {
using namespace dev;

namespace {

constexpr int kThreads = 512;

template <bool EMU> __device__ __forceinline__ const CollArgs &ArgsOf(const CollArgs &byValue, const CollArgs *emuArgs)
{
    return EMU ? emuArgs[blockIdx.y] : byValue;
}

__device__ __forceinline__ uint64_t Up128(uint64_t v) { return (v + 127) & ~127ull; }
__device__ __forceinline__ uint64_t SliceLen(uint64_t total, uint64_t slice, int j)
{
    uint64_t off = slice * (uint64_t)j;
    return off >= total ? 0 : (total - off < slice ? total - off : slice);
}

// ================================================================================================ AllReduce one-shot
// Every rank pushes its part into slot[rank] of every rank's scratch; after the channel barrier each rank reduces the
// n local slots in rank order.
template <typename T, int OP, bool EMU> __device__ void AllReduceOneShotBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    const uint64_t slot = Up128(A.bytes);
    Part p = PartOf(A.bytes, gridDim.x, blockIdx.x);
    const char *in = (const char *)A.in + p.off;
    for (int d = 0; d < n; ++d) {
        int r = (k.rank + d) % n;
        BlockCopy(k.Ccl(r) + (uint64_t)k.rank * slot + p.off, in, p.len);
    }
    if (!ChannelBarrier(k, 1)) return;
    const char *slots[kMaxRanks];
    for (int r = 0; r < n; ++r) slots[r] = k.Ccl(k.rank) + (uint64_t)r * slot + p.off;
    ReduceSlots<T, OP, kMaxRanks>((T *)((char *)A.out + p.off), (T *)nullptr, slots, n, p.len / sizeof(T));
}

// ================================================================================================ AllReduce two-shot
// Reduce-scatter by push (slice j of every rank lands in rank j's slots), ordered reduce of the own slice, all-gather
// by pull from the owners' result regions.
template <typename T, int OP> __device__ void AllReduceTwoShotCore(KCtx &k, const char *in, char *out, uint64_t bytes)
{
    const int n = k.nranks;
    const uint64_t slice = Up128((bytes + n - 1) / n);
    for (int d = 0; d < n; ++d) {
        int r = (k.rank + d) % n;
        Part p = PartOf(SliceLen(bytes, slice, r), k.vGrid, k.vBlock);
        BlockCopy(k.Ccl(r) + (uint64_t)k.rank * slice + p.off, in + (uint64_t)r * slice + p.off, p.len);
    }
    if (!ChannelBarrier(k, 1)) return;
    {
        Part p = PartOf(SliceLen(bytes, slice, k.rank), k.vGrid, k.vBlock);
        const char *slots[kMaxRanks];
        for (int r = 0; r < n; ++r) slots[r] = k.Ccl(k.rank) + (uint64_t)r * slice + p.off;
        T *res = (T *)(k.Ccl(k.rank) + (uint64_t)n * slice + p.off);
        ReduceSlots<T, OP, kMaxRanks>((T *)(out + (uint64_t)k.rank * slice + p.off), res, slots, n, p.len / sizeof(T));
    }
    if (!ChannelBarrier(k, 2)) return;
    for (int d = 1; d < n; ++d) {
        int r = (k.rank + d) % n;
        Part p = PartOf(SliceLen(bytes, slice, r), k.vGrid, k.vBlock);
        BlockCopy(out + (uint64_t)r * slice + p.off, k.Ccl(r) + (uint64_t)n * slice + p.off, p.len);
    }
}
template <typename T, int OP, bool EMU> __device__ void AllReduceTwoShotBody(KCtx &k, const CollArgs &A)
{
    AllReduceTwoShotCore<T, OP>(k, (const char *)A.in, (char *)A.out, A.bytes);
}

// ================================================================================================ AllReduce ring
// Reduce-scatter then all-gather around the ring rank -> rank + 1, one slice per step, every step into its own scratch
// slot at the receiver (2(n-1) slots, so no slot is reused inside an operator and no acknowledgements are needed). The
// comparator for the mesh kernels: same bytes per link as two-shot but 2(n-1) dependent steps instead of 2 (reference:
// docs/zh/user_guide/coll_algo_intro/Ring.md:25-31 for the cost model; HCCL's ring runs as host-issued tasks).
template <typename T, int OP> __device__ __forceinline__ void ReduceTwoTo(char *dst, char *dst2, const char *a, const char *b, uint64_t bytes)
{
    using Ac = typename Acc<T>::type;
    constexpr int VE = 16 / sizeof(T);
    const bool vecOk = ((((uintptr_t)dst | (uintptr_t)dst2 | (uintptr_t)a | (uintptr_t)b) & 15u) == 0);
    const uint64_t nvec = vecOk ? bytes >> 4 : 0;
    for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
        uint4 ra = ((const uint4 *)a)[i], rb = ((const uint4 *)b)[i], out;
        const T *ea = (const T *)&ra, *eb = (const T *)&rb;
        T *eo = (T *)&out;
#pragma unroll
        for (int j = 0; j < VE; ++j) eo[j] = FromAcc<T>(Combine<OP, Ac>(ToAcc<T>(ea[j]), ToAcc<T>(eb[j])));
        ((uint4 *)dst)[i] = out;
        if (dst2) ((uint4 *)dst2)[i] = out;
    }
    const uint64_t nElems = bytes / sizeof(T);
    for (uint64_t i = nvec * VE + threadIdx.x; i < nElems; i += blockDim.x) {
        T v = FromAcc<T>(Combine<OP, Ac>(ToAcc<T>(((const T *)a)[i]), ToAcc<T>(((const T *)b)[i])));
        ((T *)dst)[i] = v;
        if (dst2) ((T *)dst2)[i] = v;
    }
}

template <typename T, int OP, bool EMU> __device__ void AllReduceRingBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks, next = (k.rank + 1) % n, prev = (k.rank + n - 1) % n;
    const uint64_t slice = Up128((A.bytes + n - 1) / n);
    auto part = [&](int j) { return PartOf(SliceLen(A.bytes, slice, j), gridDim.x, blockIdx.x); };
    auto slot = [&](int rk, int step) { return k.Ccl(rk) + (uint64_t)step * slice; };
    const char *in = (const char *)A.in;
    char *out = (char *)A.out;
    // after all stores of the CTA: tell `next` that step `done` (1-based) has arrived in its scratch
    auto signal = [&](uint32_t done) {
        __syncthreads();
        if (threadIdx.x == 0) StReleaseSys(&FlagsOf(k.PeerHeap(next))->barrier[k.chan][k.rank], k.epoch + done);
    };
    auto waitFor = [&](uint32_t done) -> bool {
        bool mine = true;
        if (threadIdx.x == 0) mine = WaitFlagGe(k, &k.flags->barrier[k.chan][prev], k.epoch + done, (uint32_t)prev, 300u + done);
        int all = __syncthreads_and(mine ? 1 : 0);
        if (!all) k.ok = false;
        return all != 0;
    };
    // ---- reduce-scatter: at step s this rank sends (its partial of) slice (rank - s) and receives slice (rank - 1 - s)
    for (int s = 0; s < n - 1; ++s) {
        const int j = (k.rank - s + n) % n;
        Part p = part(j);
        if (s == 0) BlockCopy(slot(next, 0) + p.off, in + (uint64_t)j * slice + p.off, p.len);
        else {
            if (!waitFor((uint32_t)s)) return;
            ReduceTwoTo<T, OP>(slot(next, s) + p.off, nullptr, slot(k.rank, s - 1) + p.off, in + (uint64_t)j * slice + p.off, p.len);
        }
        signal((uint32_t)s + 1);
    }
    // ---- the last partial received is slice (rank + 1): finish it, keep it, and start the all-gather with it
    {
        if (!waitFor((uint32_t)n - 1)) return;
        const int j = (k.rank + 1) % n;
        Part p = part(j);
        ReduceTwoTo<T, OP>(out + (uint64_t)j * slice + p.off, n > 2 ? slot(next, n - 1) + p.off : nullptr, slot(k.rank, n - 2) + p.off,
                           in + (uint64_t)j * slice + p.off, p.len);
        if (n == 2) BlockCopy(slot(next, n - 1) + p.off, out + (uint64_t)j * slice + p.off, p.len);
        signal((uint32_t)n);
    }
    // ---- all-gather: step a delivers slice (rank + 1 - a); forward it unless it is the last hop
    for (int a = 1; a < n; ++a) {
        if (!waitFor((uint32_t)(n - 1 + a))) return;
        const int j = (k.rank + 1 - a + n) % n;
        Part p = part(j);
        const char *got = slot(k.rank, n - 2 + a) + p.off;
        BlockCopy(out + (uint64_t)j * slice + p.off, got, p.len);
        if (a < n - 1) {
            BlockCopy(slot(next, n - 1 + a) + p.off, got, p.len);
            signal((uint32_t)(n + a));
        }
    }
    k.syncs += (uint32_t)(2 * n - 2);
}

// ================================================================================================ AllReduce NVLS
// out[i] <- switch-reduced value; `out` may have any alignment (element-wise store then).
template <typename T> __device__ __forceinline__ void StoreVec(T *out, uint64_t vecIdx, uint4 v, bool aligned)
{
    constexpr int VE = 16 / sizeof(T);
    if (aligned) ((uint4 *)out)[vecIdx] = v;
    else {
        const T *e = (const T *)&v;
#pragma unroll
        for (int j = 0; j < VE; ++j) out[vecIdx * VE + j] = e[j];
    }
}

// Local 16-byte loads feeding multicast stores, several in flight per thread: one load per store in program order caps a
// 96-CTA grid near 500 GB/s (49 152 threads x 16 bytes per round trip of the load).
__device__ __forceinline__ void BlockMulticast(char *mc, const char *src, uint64_t nvec)
{
    constexpr int U = 8;
    if (!HCCL_RANGE_OK(mc, nvec << 4)) return;
    const uint4 *s = (const uint4 *)src;
    const uint64_t stride = (uint64_t)blockDim.x * U;
    uint64_t i = threadIdx.x;
    for (; i + (uint64_t)blockDim.x * (U - 1) < nvec; i += stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = __ldcs(s + i + (uint64_t)u * blockDim.x);
#pragma unroll
        for (int u = 0; u < U; ++u) MultimemSt16(mc + ((i + (uint64_t)u * blockDim.x) << 4), v[u]);
    }
    for (; i < nvec; i += blockDim.x) MultimemSt16(mc + (i << 4), s[i]);
}

// Switch-side reductions are long-latency loads: keep several 16-byte requests in flight per thread.
template <typename T, int OP, typename Sink> __device__ __forceinline__ void MultimemReduceLoop(const char *mc, uint64_t nvec, Sink sink)
{
    constexpr int U = 4;
    if (!HCCL_RANGE_OK(mc, nvec << 4)) return;
    const uint64_t stride = (uint64_t)blockDim.x * U;
    uint64_t i = threadIdx.x;
    for (; i + (uint64_t)blockDim.x * (U - 1) < nvec; i += stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = MultimemLdReduce<T, OP>::Ld(mc + ((i + (uint64_t)u * blockDim.x) << 4));
#pragma unroll
        for (int u = 0; u < U; ++u) sink(i + (uint64_t)u * blockDim.x, v[u]);
    }
    for (; i < nvec; i += blockDim.x) sink(i, MultimemLdReduce<T, OP>::Ld(mc + (i << 4)));
}

template <typename T, int OP, bool EMU> __device__ void AllReduceNvlsOneShotBody(KCtx &k, const CollArgs &A)
{
    Part p = PartOf(A.bytes, gridDim.x, blockIdx.x);
    BlockCopy(k.Ccl(k.rank) + p.off, (const char *)A.in + p.off, p.len);
    if (!ChannelBarrier(k, 1)) return;
    const char *mc = k.Mc() + p.off;
    T *out = (T *)((char *)A.out + p.off);
    bool aligned = ((uintptr_t)out & 15u) == 0;
    uint64_t nvec = p.len >> 4;
    MultimemReduceLoop<T, OP>(mc, nvec, [&](uint64_t i, uint4 v) { StoreVec<T>(out, i, v, aligned); });
}

template <typename T, int OP> __device__ void AllReduceNvlsTwoShotCore(KCtx &k, const char *in, char *out, uint64_t bytes)
{
    const int n = k.nranks;
    const uint64_t slice = Up128((bytes + n - 1) / n);
    const uint64_t outRegion = (uint64_t)n * slice;
    for (int j = 0; j < n; ++j) {
        Part p = PartOf(SliceLen(bytes, slice, j), k.vGrid, k.vBlock);
        BlockCopy(k.Ccl(k.rank) + (uint64_t)j * slice + p.off, in + (uint64_t)j * slice + p.off, p.len);
    }
    if (!ChannelBarrier(k, 1)) return;
    {
        Part p = PartOf(SliceLen(bytes, slice, k.rank), k.vGrid, k.vBlock);
        char *src = k.Mc() + (uint64_t)k.rank * slice + p.off;
        char *dst = k.Mc() + outRegion + (uint64_t)k.rank * slice + p.off;
        uint64_t nvec = p.len >> 4;
        MultimemReduceLoop<T, OP>(src, nvec, [&](uint64_t i, uint4 v) { MultimemSt16(dst + (i << 4), v); });
    }
    if (!ChannelBarrier(k, 2)) return;
    for (int j = 0; j < n; ++j) {
        Part p = PartOf(SliceLen(bytes, slice, j), k.vGrid, k.vBlock);
        BlockCopy(out + (uint64_t)j * slice + p.off, k.Ccl(k.rank) + outRegion + (uint64_t)j * slice + p.off, p.len);
    }
}
template <typename T, int OP, bool EMU> __device__ void AllReduceNvlsTwoShotBody(KCtx &k, const CollArgs &A)
{
    AllReduceNvlsTwoShotCore<T, OP>(k, (const char *)A.in, (char *)A.out, A.bytes);
}

// ================================================================================================ AllReduce, two algorithms side by side
// One launch, two sub-grids: CTAs [0, splitCtas) run the switch-reduced two-shot on the first splitBytes of the payload,
// the rest run the peer-store two-shot on the remainder, each in its own scratch region (the reference's concurrent
// executors split one payload between two planes by HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO; reference:
// src/ops/all_reduce/executor/ins_v2_all_reduce_concurrent_executor.cc:159,479-487). Without a multicast mapping both parts
// run the peer-store algorithm. Channels are CTA indices, so the two parts never share a flag word.
template <typename T, int OP, bool EMU, bool NVLS> __device__ void AllReduceConcurrentBody(KCtx &k, const CollArgs &A)
{
    const uint64_t bytesA = A.splitBytes;
    const uint32_t ctasA = A.splitCtas;
    const int n = k.nranks;
    if (blockIdx.x < ctasA) {
        k.vGrid = ctasA; k.vBlock = blockIdx.x; k.cclShift = 0;
        if constexpr (NVLS) AllReduceNvlsTwoShotCore<T, OP>(k, (const char *)A.in, (char *)A.out, bytesA);
        else AllReduceTwoShotCore<T, OP>(k, (const char *)A.in, (char *)A.out, bytesA);
    } else {
        k.vGrid = gridDim.x - ctasA; k.vBlock = blockIdx.x - ctasA;
        k.cclShift = 2ull * (uint64_t)n * Up128((bytesA + n - 1) / n);          // past the larger of the two layouts of part A
        AllReduceTwoShotCore<T, OP>(k, (const char *)A.in + bytesA, (char *)A.out + bytesA, A.bytes - bytesA);
    }
}
template <typename T, int OP, bool EMU> __device__ void AllReduceConcurrentNvlsBody(KCtx &k, const CollArgs &A) { AllReduceConcurrentBody<T, OP, EMU, true>(k, A); }
template <typename T, int OP, bool EMU> __device__ void AllReduceConcurrentPlainBody(KCtx &k, const CollArgs &A) { AllReduceConcurrentBody<T, OP, EMU, false>(k, A); }

// Latency end of the pull kernels: one pass in which every thread has a 16-byte load from EACH peer in flight, instead of
// one peer after the other (n - 1 dependent round trips when a CTA's share per peer is a few KB). kG bounds the registers.
constexpr int kG = 8;
constexpr uint64_t kGatherMaxBytes = 64u << 10;
__device__ __forceinline__ void GatherParts(const uint4 *const *src, uint4 *const *dst, const uint64_t *nvec, int np, uint64_t maxVec)
{
    for (uint64_t v = threadIdx.x; v < maxVec; v += blockDim.x) {
        uint4 x[kG];
#pragma unroll
        for (int d = 0; d < kG; ++d)
            if (d < np && v < nvec[d]) x[d] = src[d][v];
#pragma unroll
        for (int d = 0; d < kG; ++d)
            if (d < np && v < nvec[d]) dst[d][v] = x[d];
    }
}

// ================================================================================================ AllGather(V), pull
template <bool EMU> __device__ void AllGatherVBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    {
        Part p = PartOf(A.recvBytes[k.rank], gridDim.x, blockIdx.x);
        BlockCopy(k.Ccl(k.rank) + p.off, (const char *)A.in + p.off, p.len);
    }
    if (!ChannelBarrier(k, 1)) return;
    uint64_t maxLen = 0;
    bool vec = (((uintptr_t)A.out) & 15u) == 0;
    for (int r = 0; r < n; ++r) {
        Part p = PartOf(A.recvBytes[r], gridDim.x, blockIdx.x);
        maxLen = p.len > maxLen ? p.len : maxLen;
        vec = vec && ((p.len | p.off | A.recvOff[r]) & 15u) == 0;
    }
    if (vec && n <= kG && maxLen <= kGatherMaxBytes && HCCL_RANGE_OK(k.Ccl(k.rank), maxLen)) {
        const uint4 *src[kG];
        uint4 *dst[kG];
        uint64_t nvec[kG];
#pragma unroll
        for (int d = 1; d < kG; ++d) {
            if (d >= n) break;
            const int r = (k.rank + d) % n;
            Part p = PartOf(A.recvBytes[r], gridDim.x, blockIdx.x);
            src[d - 1] = (const uint4 *)(k.Ccl(r) + p.off);
            dst[d - 1] = (uint4 *)((char *)A.out + A.recvOff[r] + p.off);
            nvec[d - 1] = p.len >> 4;
        }
        GatherParts(src, dst, nvec, n - 1, maxLen >> 4);
    } else {
        for (int d = 1; d < n; ++d) {
            int r = (k.rank + d) % n;
            Part p = PartOf(A.recvBytes[r], gridDim.x, blockIdx.x);
            BlockCopy((char *)A.out + A.recvOff[r] + p.off, k.Ccl(r) + p.off, p.len);
        }
    }
    char *self = (char *)A.out + A.recvOff[k.rank];
    if (self != (const char *)A.in) {
        Part p = PartOf(A.recvBytes[k.rank], gridDim.x, blockIdx.x);
        BlockCopy(self + p.off, (const char *)A.in + p.off, p.len);
    }
}

// ================================================================================================ ReduceScatter(V), push
template <typename T, int OP, bool EMU> __device__ void ReduceScatterVBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    uint64_t slot = 0;
    for (int r = 0; r < n; ++r) slot = A.sendBytes[r] > slot ? A.sendBytes[r] : slot;
    slot = Up128(slot);
    for (int d = 0; d < n; ++d) {
        int r = (k.rank + d) % n;
        Part p = PartOf(A.sendBytes[r], gridDim.x, blockIdx.x);
        BlockCopy(k.Ccl(r) + (uint64_t)k.rank * slot + p.off, (const char *)A.in + A.sendOff[r] + p.off, p.len);
    }
    if (!ChannelBarrier(k, 1)) return;
    Part p = PartOf(A.sendBytes[k.rank], gridDim.x, blockIdx.x);
    const char *slots[kMaxRanks];
    for (int r = 0; r < n; ++r) slots[r] = k.Ccl(k.rank) + (uint64_t)r * slot + p.off;
    ReduceSlots<T, OP, kMaxRanks>((T *)((char *)A.out + p.off), (T *)nullptr, slots, n, p.len / sizeof(T));
}

template <typename T, int OP, bool EMU> __device__ void ReduceScatterNvlsBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    const uint64_t slot = Up128(A.sendBytes[0]);
    for (int j = 0; j < n; ++j) {
        Part p = PartOf(A.sendBytes[j], gridDim.x, blockIdx.x);
        BlockCopy(k.Ccl(k.rank) + (uint64_t)j * slot + p.off, (const char *)A.in + A.sendOff[j] + p.off, p.len);
    }
    if (!ChannelBarrier(k, 1)) return;
    Part p = PartOf(A.sendBytes[k.rank], gridDim.x, blockIdx.x);
    const char *mc = k.Mc() + (uint64_t)k.rank * slot + p.off;
    T *out = (T *)((char *)A.out + p.off);
    bool aligned = ((uintptr_t)out & 15u) == 0;
    uint64_t nvec = p.len >> 4;
    MultimemReduceLoop<T, OP>(mc, nvec, [&](uint64_t i, uint4 v) { StoreVec<T>(out, i, v, aligned); });
}

// ================================================================================================ Broadcast
template <bool EMU> __device__ void BroadcastBody(KCtx &k, const CollArgs &A)
{
    Part p = PartOf(A.bytes, gridDim.x, blockIdx.x);
    if (k.rank == (int)A.root) BlockCopy(k.Ccl(k.rank) + p.off, (const char *)A.in + p.off, p.len);
    if (!ChannelBarrier(k, 1)) return;
    if (k.rank != (int)A.root) BlockCopy((char *)A.out + p.off, k.Ccl((int)A.root) + p.off, p.len);
}

// Root multicasts once; the switch replicates to every rank's scratch, each rank copies out locally.
template <bool EMU> __device__ void BroadcastNvlsBody(KCtx &k, const CollArgs &A)
{
    Part p = PartOf(A.bytes, gridDim.x, blockIdx.x);
    if (k.rank == (int)A.root) {
        const char *src = (const char *)A.in + p.off;
        char *mc = k.Mc() + p.off;
        uint64_t nvec = p.len >> 4;
        if (((uintptr_t)src & 15u) == 0) {
            BlockMulticast(mc, src, nvec);
        } else {
            for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
                uint4 v;
                char *b = (char *)&v;
                for (int j = 0; j < 16; ++j) b[j] = src[(i << 4) + j];
                MultimemSt16(mc + (i << 4), v);
            }
        }
    }
    if (!ChannelBarrier(k, 1)) return;
    if (k.rank != (int)A.root) BlockCopy((char *)A.out + p.off, k.Ccl(k.rank) + p.off, p.len);
}

// ================================================================================================ Reduce (to root)
template <typename T, int OP, bool EMU> __device__ void ReduceBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks, root = (int)A.root;
    const uint64_t slot = Up128(A.bytes);
    Part p = PartOf(A.bytes, gridDim.x, blockIdx.x);
    BlockCopy(k.Ccl(root) + (uint64_t)k.rank * slot + p.off, (const char *)A.in + p.off, p.len);
    if (!ChannelBarrier(k, 1)) return;
    if (k.rank != root) return;
    const char *slots[kMaxRanks];
    for (int r = 0; r < n; ++r) slots[r] = k.Ccl(root) + (uint64_t)r * slot + p.off;
    ReduceSlots<T, OP, kMaxRanks>((T *)((char *)A.out + p.off), (T *)nullptr, slots, n, p.len / sizeof(T));
}

// ================================================================================================ Scatter (pull from root)
template <bool EMU> __device__ void ScatterBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks, root = (int)A.root;
    const uint64_t blockBytes = A.bytes, slot = Up128(blockBytes);
    Part p = PartOf(blockBytes, gridDim.x, blockIdx.x);
    if (k.rank == root) {
        for (int r = 0; r < n; ++r) {
            if (r == root) continue;
            BlockCopy(k.Ccl(root) + (uint64_t)r * slot + p.off, (const char *)A.in + A.sendOff[r] + p.off, p.len);
        }
    }
    if (!ChannelBarrier(k, 1)) return;
    if (k.rank == root) BlockCopy((char *)A.out + p.off, (const char *)A.in + A.sendOff[root] + p.off, p.len);
    else BlockCopy((char *)A.out + p.off, k.Ccl(root) + (uint64_t)k.rank * slot + p.off, p.len);
}

// ================================================================================================ AlltoAll(V/VC), pull
// Sender packs the segment for each peer into its own scratch and publishes the packed offsets (one copy per
// channel, so a channel barrier orders it); receivers pull their segment.
// Every pair (src -> dst) owns a fixed slot of A.slotBytes in src's scratch, at the position of dst among src's peers, so a
// receiver knows where to pull from without asking. A pair longer than its slot moves in rounds (stage, barrier, pull,
// barrier); the number of rounds has to be the same on every rank, so each rank publishes the rounds its own row and column
// need and all take the maximum. Nothing here depends on the payload fitting the scratch window.
template <bool EMU> __device__ void AlltoAllVBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    const uint64_t Q = A.slotBytes;
    uint64_t *meta = (uint64_t *)(k.Ccl(k.rank) + k.c->cclBytes - kA2aMetaBytes) + k.chan;
    uint64_t myRounds = 0;
    for (int r = 0; r < n; ++r) {
        if (r == k.rank) continue;
        const uint64_t m = A.sendBytes[r] > A.recvBytes[r] ? A.sendBytes[r] : A.recvBytes[r];
        const uint64_t need = (m + Q - 1) / Q;
        myRounds = need > myRounds ? need : myRounds;
    }
    if (threadIdx.x == 0) *(volatile uint64_t *)meta = myRounds;             // visible to the peers after the first barrier
    {
        Part p = PartOf(A.sendBytes[k.rank], gridDim.x, blockIdx.x);
        BlockCopy((char *)A.out + A.recvOff[k.rank] + p.off, (const char *)A.in + A.sendOff[k.rank] + p.off, p.len);
    }
    auto stage = [&](uint64_t t) {
        for (int r = 0; r < n; ++r) {
            if (r == k.rank) continue;
            Part p = PartOfRound(A.sendBytes[r], Q, t, gridDim.x, blockIdx.x);
            BlockCopy(k.Ccl(k.rank) + (uint64_t)(r < k.rank ? r : r - 1) * Q + p.off, (const char *)A.in + A.sendOff[r] + t * Q + p.off, p.len);
        }
    };
    stage(0);
    if (!ChannelBarrier(k, 1)) return;
    __shared__ unsigned long long rounds;
    if (threadIdx.x == 0) rounds = myRounds;
    __syncthreads();
    if ((int)threadIdx.x < n && (int)threadIdx.x != k.rank) {
        const uint64_t *peerMeta = (const uint64_t *)(k.Ccl((int)threadIdx.x) + k.c->cclBytes - kA2aMetaBytes) + k.chan;
        atomicMax(&rounds, (unsigned long long)*(const volatile uint64_t *)peerMeta);
    }
    __syncthreads();
    const uint64_t R = rounds;
    for (uint64_t t = 0; t < R; ++t) {
        if (t > 0) {
            stage(t);
            if (!ChannelBarrier(k, 1)) return;
        }
        const uint64_t lo = t * Q;
        uint64_t maxLen = 0;
        bool vec = (((uintptr_t)A.out) & 15u) == 0 && n <= kG;
        for (int r = 0; r < n; ++r) {
            if (r == k.rank) continue;
            Part p = PartOfRound(A.recvBytes[r], Q, t, gridDim.x, blockIdx.x);
            maxLen = p.len > maxLen ? p.len : maxLen;
            vec = vec && ((p.len | p.off | (A.recvOff[r] + lo)) & 15u) == 0;
        }
        if (vec && maxLen <= kGatherMaxBytes && HCCL_RANGE_OK(k.Ccl(k.rank), maxLen)) {
            const uint4 *src[kG];
            uint4 *dst[kG];
            uint64_t nvec[kG];
#pragma unroll
            for (int d = 1; d < kG; ++d) {
                if (d >= n) break;
                const int r = (k.rank + d) % n;
                Part p = PartOfRound(A.recvBytes[r], Q, t, gridDim.x, blockIdx.x);
                src[d - 1] = (const uint4 *)(k.Ccl(r) + (uint64_t)(k.rank < r ? k.rank : k.rank - 1) * Q + p.off);
                dst[d - 1] = (uint4 *)((char *)A.out + A.recvOff[r] + lo + p.off);
                nvec[d - 1] = p.len >> 4;
            }
            GatherParts(src, dst, nvec, n - 1, maxLen >> 4);
        } else {
            for (int d = 1; d < n; ++d) {
                const int r = (k.rank + d) % n;
                Part p = PartOfRound(A.recvBytes[r], Q, t, gridDim.x, blockIdx.x);
                BlockCopy((char *)A.out + A.recvOff[r] + lo + p.off, k.Ccl(r) + (uint64_t)(k.rank < r ? k.rank : k.rank - 1) * Q + p.off, p.len);
            }
        }
        if (t + 1 < R && !ChannelBarrier(k, 2)) return;          // the slots are rewritten by the next round
    }
}

// ================================================================================================ zero-copy forms
// The caller's buffers are registered windows of the symmetric heap at the same offset on every rank (HcclCommSymAlloc +
// HcclCommMemReg), so a peer's buffer is PeerHeap(r) + offset and the switch sees all of them at mcHeap + offset: nothing
// is copied into or out of the CCL scratch. Every kernel starts with a channel barrier (all ranks have entered, so their
// earlier work on these buffers is complete) and ends with one (no rank returns while a peer still reads its input or
// writes its output). HCCL's counterpart lets peers write registered user buffers directly in graph mode (reference:
// src/ops/op_common/op_common.cc:1670-1711).
template <typename T, int OP> __device__ __forceinline__ void ReduceRanksTo(KCtx &k, uint64_t srcOff, char *const *dsts, int ndst, uint64_t bytes)
{
    const char *slots[kMaxRanks];
    for (int r = 0; r < k.nranks; ++r) slots[r] = k.PeerHeap(r) + srcOff;
    for (int r = 0; r < k.nranks; ++r) if (!HCCL_RANGE_OK(slots[r], bytes)) return;
    for (int d = 0; d < ndst; ++d) if (!HCCL_RANGE_OK(dsts[d], bytes)) return;
    using Ac = typename Acc<T>::type;
    constexpr int VE = 16 / sizeof(T);
    const uint64_t nvec = bytes >> 4;
    for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
        Ac acc[VE];
        for (int r = 0; r < k.nranks; ++r) {
            uint4 raw = ((const uint4 *)slots[r])[i];
            const T *e = (const T *)&raw;
#pragma unroll
            for (int j = 0; j < VE; ++j) acc[j] = r == 0 ? ToAcc<T>(e[j]) : Combine<OP, Ac>(acc[j], ToAcc<T>(e[j]));
        }
        uint4 res;
        T *e = (T *)&res;
#pragma unroll
        for (int j = 0; j < VE; ++j) e[j] = FromAcc<T>(acc[j]);
        for (int d = 0; d < ndst; ++d) ((uint4 *)dsts[d])[i] = res;
    }
}

// in place or out of place, both windows registered; bytes a multiple of 16. Rank r owns slice r: it alone reads that slice
// of every rank's input and writes it to every rank's output, so in-place operation has no hazard.
template <typename T, int OP, bool EMU, bool NVLS> __device__ void AllReduceZcBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    const uint64_t slice = Up128((A.bytes + n - 1) / n);
    if (!ChannelBarrier(k, 1)) return;
    Part p = PartOf(SliceLen(A.bytes, slice, k.rank), k.vGrid, k.vBlock);
    const uint64_t so = (uint64_t)k.rank * slice + p.off;
    if constexpr (NVLS) {
        const char *src = k.c->mcHeap + A.inOff + so;
        char *dst = k.c->mcHeap + A.outOff + so;
        MultimemReduceLoop<T, OP>(src, p.len >> 4, [&](uint64_t i, uint4 v) { MultimemSt16(dst + (i << 4), v); });
    } else {
        char *dsts[kMaxRanks];
        for (int d = 0; d < n; ++d) dsts[d] = k.PeerHeap((k.rank + d) % n) + A.outOff + so;
        ReduceRanksTo<T, OP>(k, A.inOff + so, dsts, n, p.len);
    }
    ChannelBarrier(k, 2);
}
template <typename T, int OP, bool EMU> __device__ void AllReduceZcPlainBody(KCtx &k, const CollArgs &A) { AllReduceZcBody<T, OP, EMU, false>(k, A); }
template <typename T, int OP, bool EMU> __device__ void AllReduceZcNvlsBody(KCtx &k, const CollArgs &A) { AllReduceZcBody<T, OP, EMU, true>(k, A); }

// input window registered ([n x bytes]), output anywhere (16-byte aligned)
template <typename T, int OP, bool EMU, bool NVLS> __device__ void ReduceScatterZcBody(KCtx &k, const CollArgs &A)
{
    if (!ChannelBarrier(k, 1)) return;
    Part p = PartOf(A.bytes, k.vGrid, k.vBlock);
    const uint64_t so = (uint64_t)k.rank * A.bytes + p.off;
    char *out = (char *)A.out + p.off;
    if constexpr (NVLS) {
        T *o = (T *)out;
        MultimemReduceLoop<T, OP>(k.c->mcHeap + A.inOff + so, p.len >> 4, [&](uint64_t i, uint4 v) { ((uint4 *)o)[i] = v; });
    } else {
        char *dsts[1] = {out};
        ReduceRanksTo<T, OP>(k, A.inOff + so, dsts, 1, p.len);
    }
    ChannelBarrier(k, 2);
}
template <typename T, int OP, bool EMU> __device__ void ReduceScatterZcPlainBody(KCtx &k, const CollArgs &A) { ReduceScatterZcBody<T, OP, EMU, false>(k, A); }
template <typename T, int OP, bool EMU> __device__ void ReduceScatterZcNvlsBody(KCtx &k, const CollArgs &A) { ReduceScatterZcBody<T, OP, EMU, true>(k, A); }

// output window registered ([n x bytes]), input anywhere (16-byte aligned): every rank stores its block into every output
template <bool EMU, bool NVLS> __device__ void AllGatherZcBody(KCtx &k, const CollArgs &A)
{
    const int n = k.nranks;
    if (!ChannelBarrier(k, 1)) return;
    Part p = PartOf(A.bytes, k.vGrid, k.vBlock);
    const char *in = (const char *)A.in + p.off;
    const uint64_t doff = A.outOff + (uint64_t)k.rank * A.bytes + p.off;
    if constexpr (NVLS) {
        char *mc = k.c->mcHeap + doff;
        BlockMulticast(mc, in, p.len >> 4);
    } else {
        for (int d = 0; d < n; ++d) {
            const int r = (k.rank + d) % n;
            char *dst = k.PeerHeap(r) + doff;
            if (dst != in) BlockCopy(dst, in, p.len);
        }
    }
    ChannelBarrier(k, 2);
}
template <bool EMU> __device__ void AllGatherZcPlainBody(KCtx &k, const CollArgs &A) { AllGatherZcBody<EMU, false>(k, A); }
template <bool EMU> __device__ void AllGatherZcNvlsBody(KCtx &k, const CollArgs &A) { AllGatherZcBody<EMU, true>(k, A); }

// the buffer is a registered window on every rank: the root multicasts it (or the others pull it from the root's window)
template <bool EMU, bool NVLS> __device__ void BroadcastZcBody(KCtx &k, const CollArgs &A)
{
    if (!ChannelBarrier(k, 1)) return;
    Part p = PartOf(A.bytes, k.vGrid, k.vBlock);
    const int root = (int)A.root;
    if constexpr (NVLS) {
        if (k.rank == root) {
            const char *src = k.PeerHeap(root) + A.outOff + p.off;
            char *mc = k.c->mcHeap + A.outOff + p.off;
            BlockMulticast(mc, src, p.len >> 4);
        }
    } else if (k.rank != root) {
        BlockCopy(k.PeerHeap(k.rank) + A.outOff + p.off, k.PeerHeap(root) + A.outOff + p.off, p.len);
    }
    ChannelBarrier(k, 2);
}
template <bool EMU> __device__ void BroadcastZcPlainBody(KCtx &k, const CollArgs &A) { BroadcastZcBody<EMU, false>(k, A); }
template <bool EMU> __device__ void BroadcastZcNvlsBody(KCtx &k, const CollArgs &A) { BroadcastZcBody<EMU, true>(k, A); }

#include "pipelined.cuh"

// ================================================================================================ kernels
#define COLL_KERNEL_TYPED(NAME, BODY)                                                                                  \
    template <typename T, bool EMU>                                                                                    \
    __global__ void __launch_bounds__(kThreads) NAME(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *emuArgs) \
    {                                                                                                                  \
        KCtx k = EnterCollective<EMU>(comms);                                                                          \
        const CollArgs &A = ArgsOf<EMU>(a, emuArgs);                                                                   \
        switch (A.op) {                                                                                                \
            case HCCL_REDUCE_SUM: BODY<T, HCCL_REDUCE_SUM, EMU>(k, A); break;                                          \
            case HCCL_REDUCE_PROD: BODY<T, HCCL_REDUCE_PROD, EMU>(k, A); break;                                        \
            case HCCL_REDUCE_MAX: BODY<T, HCCL_REDUCE_MAX, EMU>(k, A); break;                                          \
            default: BODY<T, HCCL_REDUCE_MIN, EMU>(k, A); break;                                                       \
        }                                                                                                              \
        LeaveCollective(k);                                                                                            \
    }
COLL_KERNEL_TYPED(KAllReduceOneShot, AllReduceOneShotBody)
COLL_KERNEL_TYPED(KAllReduceTwoShot, AllReduceTwoShotBody)
COLL_KERNEL_TYPED(KReduceScatterV, ReduceScatterVBody)
COLL_KERNEL_TYPED(KReduce, ReduceBody)
template <typename T, int OP, bool EMU> __device__ void AllReducePipePlainBody(KCtx &k, const CollArgs &A) { pipe::AllReduceBody<T, OP, EMU, false>(k, A); }
template <typename T, int OP, bool EMU> __device__ void AllReducePipeNvlsBody(KCtx &k, const CollArgs &A) { pipe::AllReduceBody<T, OP, EMU, true>(k, A); }
template <typename T, int OP, bool EMU> __device__ void ReduceScatterPipePlainBody(KCtx &k, const CollArgs &A) { pipe::ReduceScatterBody<T, OP, EMU, false>(k, A); }
template <typename T, int OP, bool EMU> __device__ void ReduceScatterPipeNvlsBody(KCtx &k, const CollArgs &A) { pipe::ReduceScatterBody<T, OP, EMU, true>(k, A); }
template <bool EMU> __device__ void AllGatherPipePlainBody(KCtx &k, const CollArgs &A) { pipe::AllGatherBody<EMU, false>(k, A); }
template <bool EMU> __device__ void AllGatherPipeNvlsBody(KCtx &k, const CollArgs &A) { pipe::AllGatherBody<EMU, true>(k, A); }
template <bool EMU> __device__ void AlltoAllPipeBody(KCtx &k, const CollArgs &A) { pipe::AllGatherBody<EMU, false, true>(k, A); }
COLL_KERNEL_TYPED(KAllReduceRing, AllReduceRingBody)
COLL_KERNEL_TYPED(KAllReduceConcurrentPlain, AllReduceConcurrentPlainBody)
COLL_KERNEL_TYPED(KAllReduceZc, AllReduceZcPlainBody)
COLL_KERNEL_TYPED(KReduceScatterZc, ReduceScatterZcPlainBody)
COLL_KERNEL_TYPED(KAllReducePipe, AllReducePipePlainBody)
COLL_KERNEL_TYPED(KReduceScatterPipe, ReduceScatterPipePlainBody)

#define COLL_KERNEL_NVLS(NAME, BODY)                                                                                   \
    template <typename T, int OP, bool EMU>                                                                            \
    __global__ void __launch_bounds__(kThreads) NAME(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *emuArgs) \
    {                                                                                                                  \
        KCtx k = EnterCollective<EMU>(comms);                                                                          \
        BODY<T, OP, EMU>(k, ArgsOf<EMU>(a, emuArgs));                                                                  \
        LeaveCollective(k);                                                                                            \
    }
COLL_KERNEL_NVLS(KAllReduceNvlsOneShot, AllReduceNvlsOneShotBody)
COLL_KERNEL_NVLS(KAllReduceNvlsTwoShot, AllReduceNvlsTwoShotBody)
COLL_KERNEL_NVLS(KReduceScatterNvls, ReduceScatterNvlsBody)
COLL_KERNEL_NVLS(KAllReducePipeNvls, AllReducePipeNvlsBody)
COLL_KERNEL_NVLS(KAllReduceConcurrentNvls, AllReduceConcurrentNvlsBody)
COLL_KERNEL_NVLS(KAllReduceZcNvls, AllReduceZcNvlsBody)
COLL_KERNEL_NVLS(KReduceScatterZcNvls, ReduceScatterZcNvlsBody)
COLL_KERNEL_NVLS(KReduceScatterPipeNvls, ReduceScatterPipeNvlsBody)

#define COLL_KERNEL_BYTES(NAME, BODY)                                                                                  \
    template <bool EMU>                                                                                                \
    __global__ void __launch_bounds__(kThreads) NAME(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *emuArgs) \
    {                                                                                                                  \
        KCtx k = EnterCollective<EMU>(comms);                                                                          \
        BODY<EMU>(k, ArgsOf<EMU>(a, emuArgs));                                                                         \
        LeaveCollective(k);                                                                                            \
    }
COLL_KERNEL_BYTES(KAllGatherV, AllGatherVBody)
COLL_KERNEL_BYTES(KBroadcast, BroadcastBody)
COLL_KERNEL_BYTES(KBroadcastNvls, BroadcastNvlsBody)
COLL_KERNEL_BYTES(KScatter, ScatterBody)
COLL_KERNEL_BYTES(KAlltoAllV, AlltoAllVBody)
COLL_KERNEL_BYTES(KAllGatherPipe, AllGatherPipePlainBody)
COLL_KERNEL_BYTES(KAllGatherPipeNvls, AllGatherPipeNvlsBody)
COLL_KERNEL_BYTES(KAlltoAllPipe, AlltoAllPipeBody)
COLL_KERNEL_BYTES(KAllGatherZc, AllGatherZcPlainBody)
COLL_KERNEL_BYTES(KAllGatherZcNvls, AllGatherZcNvlsBody)
COLL_KERNEL_BYTES(KBroadcastZc, BroadcastZcPlainBody)
COLL_KERNEL_BYTES(KBroadcastZcNvls, BroadcastZcNvlsBody)

template <bool EMU> __global__ void __launch_bounds__(kThreads) KBarrier(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *)
{
    KCtx k = EnterCollective<EMU>(comms);
    ChannelBarrier(k, 1);
    LeaveCollective(k);
}

// ================================================================================================ point to point
// Mailbox protocol. The sender stages round m (1-based, cumulative per (peer, CTA)) in slot (m-1)&1 of its own
// mailbox for that peer and raises data[src][cta][slot] = m at the receiver; the receiver pulls and raises
// ack[dst][cta][slot] = m at the sender. A slot is refilled only after the round that used it two rounds earlier was
// acknowledged, and a send returns only when all its rounds were acknowledged (rendezvous semantics, like
// HCCL's send/recv kernels which stage into the CCL buffer and wait for the receiver's ack).
struct P2pCtx {
    const DevComm *c;
    int rank;
    char *heap;
    DevCtrl *ctrl;
    DevFlags *flags;
    KCtx k;   // for the bounded waits / reporting
};
template <bool EMU> __device__ __forceinline__ P2pCtx EnterP2p(const DevComm *comms, uint32_t chan)
{
    P2pCtx x;
    x.c = EMU ? &comms[blockIdx.y] : comms;
    x.rank = x.c->rank;
    x.heap = x.c->heap[x.rank];
    x.ctrl = CtrlOf(x.heap);
    x.flags = FlagsOf(x.heap);
    x.k.c = x.c; x.k.rank = x.rank; x.k.nranks = x.c->nranks; x.k.heap = x.heap; x.k.ctrl = x.ctrl; x.k.flags = x.flags;
    x.k.half = 0; x.k.chan = chan; x.k.epoch = 0; x.k.syncs = 0; x.k.ok = true;
    return x;
}

// cta = index within the 8 CTAs of this transfer
__device__ bool SendBody(P2pCtx &x, const char *src, uint64_t bytes, int dst, int cta)
{
    const uint64_t W = x.c->mailboxBytes, sub = W / kP2pBlocks;
    uint64_t rounds = (bytes + W - 1) / W;
    uint64_t base = x.ctrl->p2pSendSeq[dst][cta];
    bool ok = true;
    for (uint64_t r = 0; r < rounds && ok; ++r) {
        uint64_t m = base + r + 1;
        uint32_t slot = (uint32_t)((m - 1) & 1);
        if (m > 2) {
            if (threadIdx.x == 0) ok = WaitFlagGe64(x.k, &x.flags->p2pAck[dst][cta * 2 + slot], m - 2, (uint32_t)dst, 11);
            ok = __syncthreads_and(ok ? 1 : 0) != 0;
            if (!ok) break;
        }
        uint64_t chunk = bytes - r * W < W ? bytes - r * W : W;
        Part p = PartOf(chunk, kP2pBlocks, cta);
        (void)sub;
        BlockCopy(x.heap + x.c->mailboxOff + ((uint64_t)dst * 2 + slot) * W + p.off, src + r * W + p.off, p.len);
        __syncthreads();
        if (threadIdx.x == 0) StReleaseSys64(&FlagsOf(x.c->heap[dst])->p2pData[x.rank][cta * 2 + slot], m);
    }
    // all rounds acknowledged before the send completes
    if (ok && rounds > 0) {
        uint64_t last = base + rounds;
        if (threadIdx.x == 0) {
            ok = WaitFlagGe64(x.k, &x.flags->p2pAck[dst][cta * 2 + (uint32_t)((last - 1) & 1)], last, (uint32_t)dst, 12);
            if (ok && last >= 2) ok = WaitFlagGe64(x.k, &x.flags->p2pAck[dst][cta * 2 + (uint32_t)((last - 2) & 1)], last - 1, (uint32_t)dst, 13);
        }
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) x.ctrl->p2pSendSeq[dst][cta] = base + rounds;
    return ok;
}

__device__ bool RecvBody(P2pCtx &x, char *dstBuf, uint64_t bytes, int src, int cta)
{
    const uint64_t W = x.c->mailboxBytes;
    uint64_t rounds = (bytes + W - 1) / W;
    uint64_t base = x.ctrl->p2pRecvSeq[src][cta];
    bool ok = true;
    for (uint64_t r = 0; r < rounds && ok; ++r) {
        uint64_t m = base + r + 1;
        uint32_t slot = (uint32_t)((m - 1) & 1);
        if (threadIdx.x == 0) ok = WaitFlagGe64(x.k, &x.flags->p2pData[src][cta * 2 + slot], m, (uint32_t)src, 21);
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
        if (!ok) break;
        uint64_t chunk = bytes - r * W < W ? bytes - r * W : W;
        Part p = PartOf(chunk, kP2pBlocks, cta);
        BlockCopy(dstBuf + r * W + p.off, x.c->heap[src] + x.c->mailboxOff + ((uint64_t)x.rank * 2 + slot) * W + p.off, p.len);
        __syncthreads();
        if (threadIdx.x == 0) StReleaseSys64(&FlagsOf(x.c->heap[src])->p2pAck[x.rank][cta * 2 + slot], m);
    }
    __syncthreads();
    if (threadIdx.x == 0) x.ctrl->p2pRecvSeq[src][cta] = base + rounds;
    return ok;
}

template <bool EMU> __global__ void __launch_bounds__(kThreads) KSend(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *emuArgs)
{
    const CollArgs &A = ArgsOf<EMU>(a, emuArgs);
    P2pCtx x = EnterP2p<EMU>(comms, blockIdx.x);
    if (EMU && A.count == 0) return;   // emulation: ranks that do not take part
    SendBody(x, (const char *)A.in, A.bytes, (int)A.peer, (int)blockIdx.x);
}
template <bool EMU> __global__ void __launch_bounds__(kThreads) KRecv(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *emuArgs)
{
    const CollArgs &A = ArgsOf<EMU>(a, emuArgs);
    P2pCtx x = EnterP2p<EMU>(comms, blockIdx.x);
    if (EMU && A.count == 0) return;
    RecvBody(x, (char *)A.out, A.bytes, (int)A.peer, (int)blockIdx.x);
}
// Emulation only: rank A.root sends to rank A.peer inside one launch (flags 1 = sender, 2 = receiver in A.op).
template <bool EMU> __global__ void __launch_bounds__(kThreads) KSendRecvPair(const DevComm *comms, const __grid_constant__ CollArgs a, const CollArgs *emuArgs)
{
    const CollArgs &A = ArgsOf<EMU>(a, emuArgs);
    P2pCtx x = EnterP2p<EMU>(comms, blockIdx.x);
    if (A.op == 1) SendBody(x, (const char *)A.in, A.bytes, (int)A.peer, (int)blockIdx.x);
    else if (A.op == 2) RecvBody(x, (char *)A.out, A.bytes, (int)A.peer, (int)blockIdx.x);
}

// Queue q (one per (peer, direction), CTAs q*8..q*8+7) walks its items in order; queues run concurrently, so no
// ordering of unrelated pairs can deadlock.
template <bool EMU> __global__ void __launch_bounds__(kThreads) KBatchSendRecv(const DevComm *comms, const __grid_constant__ BatchArgs b, const BatchArgs *emuBatch)
{
    const BatchArgs &B = EMU ? emuBatch[blockIdx.y] : b;
    uint32_t queue = blockIdx.x / kP2pBlocks, cta = blockIdx.x % kP2pBlocks;
    if (queue >= B.nQueues) return;
    P2pCtx x = EnterP2p<EMU>(comms, blockIdx.x);
    uint32_t nInQueue = 0;
    for (uint32_t i = 0; i < B.nItems; ++i) if (B.items[i].queue == queue) ++nInQueue;
    for (uint32_t ord = 0; ord < nInQueue; ++ord) {
        for (uint32_t i = 0; i < B.nItems; ++i) {
            const BatchItem &it = B.items[i];
            if (it.queue != queue || it.order != ord) continue;
            bool ok = true;
            if (it.isSend == 1) ok = SendBody(x, (const char *)it.buf, it.bytes, (int)it.peer, (int)cta);
            else if (it.isSend == 0) ok = RecvBody(x, (char *)it.buf, it.bytes, (int)it.peer, (int)cta);
            else { Part p = PartOf(it.bytes, kP2pBlocks, cta); BlockCopy((char *)it.buf2 + p.off, (const char *)it.buf + p.off, p.len); }
            if (!ok) return;
        }
    }
}

// ---------------------------------------------------------------------------------------------- launch tables
using CollKernelFn = void (*)(const DevComm *, const CollArgs, const CollArgs *);

template <bool EMU> CollKernelFn TypedKernel(SmKernelId id, HcclDataType dt)
{
#define PICK(KERN)                                                                 \
    switch (dt) {                                                                  \
        case HCCL_DATA_TYPE_INT8: return KERN<int8_t, EMU>;                        \
        case HCCL_DATA_TYPE_INT16: return KERN<int16_t, EMU>;                      \
        case HCCL_DATA_TYPE_INT32: return KERN<int32_t, EMU>;                      \
        case HCCL_DATA_TYPE_INT64: return KERN<long long, EMU>;                    \
        case HCCL_DATA_TYPE_UINT64: return KERN<unsigned long long, EMU>;          \
        case HCCL_DATA_TYPE_UINT8: return KERN<uint8_t, EMU>;                      \
        case HCCL_DATA_TYPE_UINT16: return KERN<uint16_t, EMU>;                    \
        case HCCL_DATA_TYPE_UINT32: return KERN<uint32_t, EMU>;                    \
        case HCCL_DATA_TYPE_FP16: return KERN<__half, EMU>;                        \
        case HCCL_DATA_TYPE_FP32: return KERN<float, EMU>;                         \
        case HCCL_DATA_TYPE_FP64: return KERN<double, EMU>;                        \
        case HCCL_DATA_TYPE_BFP16: return KERN<__nv_bfloat16, EMU>;                \
        default: return nullptr;                                                   \
    }
    switch (id) {
        case K_ALLREDUCE_ONESHOT: PICK(KAllReduceOneShot)
        case K_ALLREDUCE_TWOSHOT: PICK(KAllReduceTwoShot)
        case K_REDUCESCATTER_V: PICK(KReduceScatterV)
        case K_REDUCE: PICK(KReduce)
        case K_ALLREDUCE_RING: PICK(KAllReduceRing)
        case K_ALLREDUCE_CONCURRENT: PICK(KAllReduceConcurrentPlain)
        case K_ALLREDUCE_ZC: PICK(KAllReduceZc)
        case K_REDUCESCATTER_ZC: PICK(KReduceScatterZc)
        case K_ALLREDUCE_PIPE: PICK(KAllReducePipe)
        case K_REDUCESCATTER_PIPE: PICK(KReduceScatterPipe)
        default: return nullptr;
    }
#undef PICK
}

template <bool EMU> CollKernelFn NvlsKernel(SmKernelId id, HcclDataType dt, HcclReduceOp op)
{
#define PICKN(KERN)                                                                                         \
    if (dt == HCCL_DATA_TYPE_FP32 && op == HCCL_REDUCE_SUM) return KERN<float, HCCL_REDUCE_SUM, EMU>;       \
    if (dt == HCCL_DATA_TYPE_BFP16 && op == HCCL_REDUCE_SUM) return KERN<__nv_bfloat16, HCCL_REDUCE_SUM, EMU>; \
    if (dt == HCCL_DATA_TYPE_BFP16 && op == HCCL_REDUCE_MAX) return KERN<__nv_bfloat16, HCCL_REDUCE_MAX, EMU>; \
    if (dt == HCCL_DATA_TYPE_BFP16 && op == HCCL_REDUCE_MIN) return KERN<__nv_bfloat16, HCCL_REDUCE_MIN, EMU>; \
    if (dt == HCCL_DATA_TYPE_FP16 && op == HCCL_REDUCE_SUM) return KERN<__half, HCCL_REDUCE_SUM, EMU>;      \
    if (dt == HCCL_DATA_TYPE_FP16 && op == HCCL_REDUCE_MAX) return KERN<__half, HCCL_REDUCE_MAX, EMU>;      \
    if (dt == HCCL_DATA_TYPE_FP16 && op == HCCL_REDUCE_MIN) return KERN<__half, HCCL_REDUCE_MIN, EMU>;      \
    return nullptr;
    switch (id) {
        case K_ALLREDUCE_NVLS_ONESHOT: PICKN(KAllReduceNvlsOneShot)
        case K_ALLREDUCE_NVLS_TWOSHOT: PICKN(KAllReduceNvlsTwoShot)
        case K_REDUCESCATTER_NVLS: PICKN(KReduceScatterNvls)
        case K_ALLREDUCE_PIPE_NVLS: PICKN(KAllReducePipeNvls)
        case K_ALLREDUCE_CONCURRENT_NVLS: PICKN(KAllReduceConcurrentNvls)
        case K_ALLREDUCE_ZC_NVLS: PICKN(KAllReduceZcNvls)
        case K_REDUCESCATTER_ZC_NVLS: PICKN(KReduceScatterZcNvls)
        case K_REDUCESCATTER_PIPE_NVLS: PICKN(KReduceScatterPipeNvls)
        default: return nullptr;
    }
#undef PICKN
}

template <bool EMU> CollKernelFn KernelFor(const SmLaunch &l)
{
    switch (l.kernel) {
        case K_ALLREDUCE_ONESHOT: case K_ALLREDUCE_TWOSHOT: case K_REDUCESCATTER_V: case K_REDUCE: case K_ALLREDUCE_PIPE: case K_REDUCESCATTER_PIPE: case K_ALLREDUCE_RING: case K_ALLREDUCE_CONCURRENT: case K_ALLREDUCE_ZC: case K_REDUCESCATTER_ZC:
            return TypedKernel<EMU>(l.kernel, l.dtype);
        case K_ALLREDUCE_NVLS_ONESHOT: case K_ALLREDUCE_NVLS_TWOSHOT: case K_REDUCESCATTER_NVLS: case K_ALLREDUCE_PIPE_NVLS: case K_REDUCESCATTER_PIPE_NVLS: case K_ALLREDUCE_CONCURRENT_NVLS: case K_ALLREDUCE_ZC_NVLS: case K_REDUCESCATTER_ZC_NVLS:
            return NvlsKernel<EMU>(l.kernel, l.dtype, (HcclReduceOp)l.args.op);
        case K_ALLGATHER_PIPE: return KAllGatherPipe<EMU>;
        case K_ALLGATHER_PIPE_NVLS: return KAllGatherPipeNvls<EMU>;
        case K_ALLTOALL_PIPE: return KAlltoAllPipe<EMU>;
        case K_ALLGATHER_ZC: return KAllGatherZc<EMU>;
        case K_ALLGATHER_ZC_NVLS: return KAllGatherZcNvls<EMU>;
        case K_BROADCAST_ZC: return KBroadcastZc<EMU>;
        case K_BROADCAST_ZC_NVLS: return KBroadcastZcNvls<EMU>;
        case K_ALLGATHER_V: return KAllGatherV<EMU>;
        case K_BROADCAST: return KBroadcast<EMU>;
        case K_BROADCAST_NVLS: return KBroadcastNvls<EMU>;
        case K_SCATTER: return KScatter<EMU>;
        case K_ALLTOALL_V: return KAlltoAllV<EMU>;
        case K_BARRIER: return KBarrier<EMU>;
        case K_SEND: return KSend<EMU>;
        case K_RECV: return KRecv<EMU>;
        default: return nullptr;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------- host entry points
HcclResult SmIssueLaunch(const DevComm *devComm, const SmLaunch &l, cudaStream_t stream)
{
    if (l.kernel == K_BATCH_SEND_RECV) {
        KBatchSendRecv<false><<<l.ctas, kThreads, 0, stream>>>(devComm, l.batch, nullptr);
    } else {
        CollKernelFn fn = KernelFor<false>(l);
        if (!fn) return HCCL_E_NOT_SUPPORT;
        fn<<<l.ctas, kThreads, 0, stream>>>(devComm, l.args, nullptr);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

// Emulation: one cooperative launch covers all ranks (grid = ctas x nranks); argument blocks come from device memory.
HcclResult SmIssueEmuLaunch(const DevComm *devComms, int nranks, const SmLaunch &l0, const CollArgs *devArgs, const BatchArgs *devBatch,
                            cudaStream_t stream, bool pairKernel)
{
    dim3 grid(l0.ctas, nranks), block(kThreads);
    cudaError_t e;
    if (l0.kernel == K_BATCH_SEND_RECV) {
        BatchArgs dummyB = l0.batch;
        void *params[] = {(void *)&devComms, (void *)&dummyB, (void *)&devBatch};
        e = cudaLaunchCooperativeKernel((void *)KBatchSendRecv<true>, grid, block, params, 0, stream);
    } else {
        CollKernelFn fn = pairKernel ? (CollKernelFn)KSendRecvPair<true> : KernelFor<true>(l0);
        if (!fn) return HCCL_E_NOT_SUPPORT;
        CollArgs dummy = l0.args;
        void *params[] = {(void *)&devComms, (void *)&dummy, (void *)&devArgs};
        e = cudaLaunchCooperativeKernel((void *)fn, grid, block, params, 0, stream);
    }
    if (e != cudaSuccess) return e == cudaErrorCooperativeLaunchTooLarge ? HCCL_E_PARA : HCCL_E_RUNTIME;
    return HCCL_SUCCESS;
}

}  // namespace hccl
