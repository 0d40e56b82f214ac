// Warp-specialised, software-pipelined collectives for payloads of any size in ONE launch.
//
// The plain kernels of collectives.cu run "stage in -> synchronise -> move over NVLink -> synchronise -> copy out" as
// consecutive phases of the whole CTA, so the local staging copies and the NVLink traffic never overlap and the payload
// of a launch is bounded by the scratch size. Here the CTA's warps split into role groups that work on different
// sub-chunks at the same time, connected by counting flags in the symmetric heap:
//
//   stagers    user input   -> staging ring slot d = c % depth (local HBM copy)            signal STAGED  = c+1
//   movers     NVLS: multimem.ld_reduce of the own slice over all ranks' slot d, multimem.st of the result into every
//              rank's result ring; plain: ordered reduce over peer loads, peer stores      signal MOVED   = c+1
//   drainers   result ring slot d -> user output (local HBM copy)                          signal DRAINED = c+1
//
// A ring slot is reused once every rank has signalled the flag that ends its use (stagers wait MOVED c-depth, movers
// wait DRAINED c-depth). Flags only grow; the per-channel base lives in the control block, so captured graphs replay.
// Every wait is bounded: on expiry the role records the timeout, raises the abort flag and all roles leave.
//
// HCCL's closest relative is the multi-core pipelining of its vector-core two-shot kernel (reference:
// src/ops/all_reduce/template/aiv/kernel/aiv_all_reduce_mesh_1d_twoshot.h:16-349, cores split into senders / reducers /
// gatherers with per-slice flags); the NVLS movers have no counterpart there.
#pragma once

namespace pipe {

constexpr int kDepth = 2;
enum Flag : int { STAGED = 0, MOVED = 1, DRAINED = 2 };

struct Role {
    int tid, nthr, bar;       // thread index within the group, group size, named barrier id (1..15)
};

__device__ __forceinline__ void BarSync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// All ranks (this one included) have raised `kind` on this channel to `target`. Whole group calls; false = give up.
__device__ __forceinline__ bool Wait(KCtx &k, const Role &r, int kind, uint32_t target, int *sFail)
{
    if (r.tid < k.nranks) {
        if (!WaitFlagGe(k, &k.flags->pipe[kind][k.chan][r.tid], target, (uint32_t)r.tid, 200u + (uint32_t)kind)) atomicExch(sFail, 1);
    }
    BarSync(r.bar, r.nthr);
    return *(volatile int *)sFail == 0;
}

// Publishes `value` for `kind` to every rank after all stores of the group have been issued.
__device__ __forceinline__ void Signal(KCtx &k, const Role &r, int kind, uint32_t value)
{
    BarSync(r.bar, r.nthr);
    if (r.tid < k.nranks) StReleaseSys(&FlagsOf(k.PeerHeap(r.tid))->pipe[kind][k.chan][k.rank], value);
}

// Copy by one role group. 16-byte vectors with 8 loads in flight per thread when both sides are aligned.
__device__ __forceinline__ void Copy(void *dst, const void *src, uint64_t n, const Role &r)
{
    if (n == 0) return;
    HCCL_CHECK_RANGE(dst, src, n);
    uintptr_t a = (uintptr_t)dst | (uintptr_t)src;
    if ((a & 15u) == 0) {
        constexpr int U = 8;
        const uint4 *s = (const uint4 *)src;
        uint4 *d = (uint4 *)dst;
        uint64_t nvec = n >> 4, i = r.tid;
        const uint64_t stride = (uint64_t)r.nthr * U;
        for (; i + (uint64_t)r.nthr * (U - 1) < nvec; i += stride) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = s[i + (uint64_t)u * r.nthr];
#pragma unroll
            for (int u = 0; u < U; ++u) d[i + (uint64_t)u * r.nthr] = v[u];
        }
        for (; i < nvec; i += r.nthr) d[i] = s[i];
        for (uint64_t b = (nvec << 4) + r.tid; b < n; b += r.nthr) ((char *)dst)[b] = ((const char *)src)[b];
    } else if ((a & 3u) == 0) {
        uint64_t nw = n >> 2;
        for (uint64_t i = r.tid; i < nw; i += r.nthr) ((uint32_t *)dst)[i] = ((const uint32_t *)src)[i];
        for (uint64_t b = (nw << 2) + r.tid; b < n; b += r.nthr) ((char *)dst)[b] = ((const char *)src)[b];
    } else {
        for (uint64_t b = r.tid; b < n; b += r.nthr) ((char *)dst)[b] = ((const char *)src)[b];
    }
}

// Geometry shared by the three operators: this channel's window of every ring slot.
struct Geo {
    int n, G, ch;
    uint64_t sub;         // bytes of one sub-chunk per (slice, channel)
    uint32_t chunks;      // sub-chunks this channel walks through
    uint32_t base;        // flag value before this operator
    __device__ __forceinline__ uint64_t Slot(int d, int j) const { return (((uint64_t)d * n + j) * G + ch) * sub; }
    __device__ __forceinline__ uint64_t RingBytes() const { return (uint64_t)kDepth * n * G * sub; }
};

__device__ __forceinline__ Geo MakeGeo(KCtx &k, const CollArgs &A, uint64_t longestPart)
{
    Geo g;
    g.n = k.nranks;
    g.G = (int)gridDim.x;
    g.ch = (int)blockIdx.x;
    g.sub = A.pipeSub;
    g.chunks = (uint32_t)((longestPart + g.sub - 1) / g.sub);
    g.base = LdVolatile(&k.ctrl->pipeEpoch[g.ch]);
    return g;
}

// Length of sub-chunk c inside a part of `len` bytes.
__device__ __forceinline__ uint64_t SubLen(uint64_t len, uint64_t sub, uint32_t c)
{
    uint64_t lo = (uint64_t)c * sub;
    return lo >= len ? 0 : (len - lo < sub ? len - lo : sub);
}

// Every role has finished: advance the channel's flag base for the next operator.
__device__ __forceinline__ void Finish(KCtx &k, const Geo &g)
{
    __syncthreads();
    if (threadIdx.x == 0) *((volatile uint32_t *)&k.ctrl->pipeEpoch[g.ch]) = g.base + g.chunks;
}

// ---------------------------------------------------------------------------------------------- movers
// NVLS: result of the switch-side reduction over all ranks' slot, multicast back into every rank's result ring.
template <typename T, int OP> __device__ __forceinline__ void MoveReduceNvls(const char *mcSrc, char *mcDst, uint64_t bytes, const Role &r)
{
    constexpr int U = 8;
    uint64_t nvec = bytes >> 4, i = r.tid;
    const uint64_t stride = (uint64_t)r.nthr * U;
    for (; i + (uint64_t)r.nthr * (U - 1) < nvec; i += stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = MultimemLdReduce<T, OP>::Ld(mcSrc + ((i + (uint64_t)u * r.nthr) << 4));
#pragma unroll
        for (int u = 0; u < U; ++u) MultimemSt16(mcDst + ((i + (uint64_t)u * r.nthr) << 4), v[u]);
    }
    for (; i < nvec; i += r.nthr) MultimemSt16(mcDst + (i << 4), MultimemLdReduce<T, OP>::Ld(mcSrc + (i << 4)));
}

// NVLS reduce straight into (local) user memory: ReduceScatter.
template <typename T, int OP> __device__ __forceinline__ void MoveReduceNvlsToLocal(const char *mcSrc, T *out, uint64_t bytes, const Role &r)
{
    constexpr int U = 8;
    const bool aligned = ((uintptr_t)out & 15u) == 0;
    uint64_t nvec = bytes >> 4, i = r.tid;
    const uint64_t stride = (uint64_t)r.nthr * U;
    for (; i + (uint64_t)r.nthr * (U - 1) < nvec; i += stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = MultimemLdReduce<T, OP>::Ld(mcSrc + ((i + (uint64_t)u * r.nthr) << 4));
#pragma unroll
        for (int u = 0; u < U; ++u) StoreVec<T>(out, i + (uint64_t)u * r.nthr, v[u], aligned);
    }
    for (; i < nvec; i += r.nthr) StoreVec<T>(out, i, MultimemLdReduce<T, OP>::Ld(mcSrc + (i << 4)), aligned);
}

// Plain peer memory: rank-ordered reduction over the n ranks' slots; the result goes to `nDst` destinations
// (every rank's result ring for AllReduce, the local user buffer for ReduceScatter). Slots are 16-byte aligned.
template <typename T, int OP>
__device__ __forceinline__ void MoveReducePlain(const char *const *src, int nsrc, char *const *dst, int ndst, uint64_t bytes, const Role &r)
{
    using A = typename Acc<T>::type;
    constexpr int VE = 16 / sizeof(T);
    bool vecOk = true;
    for (int q = 0; q < ndst; ++q) vecOk = vecOk && (((uintptr_t)dst[q] & 15u) == 0);
    uint64_t nvec = vecOk ? bytes >> 4 : 0;
    // two vectors per thread and iteration: 2 x nsrc independent 16-byte loads in flight before the first use
    constexpr int U = 2;
    uint64_t i = r.tid;
    for (; i + (uint64_t)r.nthr * (U - 1) < nvec; i += (uint64_t)r.nthr * U) {
        uint4 raw[U][kMaxRanks > 8 ? 8 : kMaxRanks];
        A acc[U][VE];
        for (int s0 = 0; s0 < nsrc; s0 += 8) {
            const int ns = nsrc - s0 < 8 ? nsrc - s0 : 8;
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < ns) raw[u][s] = ((const uint4 *)src[s0 + s])[i + (uint64_t)u * r.nthr];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    if (s >= ns) continue;
                    const T *e = (const T *)&raw[u][s];
#pragma unroll
                    for (int j = 0; j < VE; ++j) acc[u][j] = (s0 + s == 0) ? ToAcc<T>(e[j]) : Combine<OP, A>(acc[u][j], ToAcc<T>(e[j]));
                }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint4 res;
            T *e = (T *)&res;
#pragma unroll
            for (int j = 0; j < VE; ++j) e[j] = FromAcc<T>(acc[u][j]);
            for (int q = 0; q < ndst; ++q) ((uint4 *)dst[q])[i + (uint64_t)u * r.nthr] = res;
        }
    }
    for (; i < nvec; i += r.nthr) {
        A acc[VE];
        {
            uint4 raw = ((const uint4 *)src[0])[i];
            const T *e = (const T *)&raw;
#pragma unroll
            for (int j = 0; j < VE; ++j) acc[j] = ToAcc<T>(e[j]);
        }
        for (int s = 1; s < nsrc; ++s) {
            uint4 raw = ((const uint4 *)src[s])[i];
            const T *e = (const T *)&raw;
#pragma unroll
            for (int j = 0; j < VE; ++j) acc[j] = Combine<OP, A>(acc[j], ToAcc<T>(e[j]));
        }
        uint4 res;
        T *e = (T *)&res;
#pragma unroll
        for (int j = 0; j < VE; ++j) e[j] = FromAcc<T>(acc[j]);
        for (int q = 0; q < ndst; ++q) ((uint4 *)dst[q])[i] = res;
    }
    const uint64_t nElems = bytes / sizeof(T);
    for (uint64_t i = nvec * VE + r.tid; i < nElems; i += r.nthr) {
        A acc = ToAcc<T>(((const T *)src[0])[i]);
        for (int s = 1; s < nsrc; ++s) acc = Combine<OP, A>(acc, ToAcc<T>(((const T *)src[s])[i]));
        T v = FromAcc<T>(acc);
        for (int q = 0; q < ndst; ++q) ((T *)dst[q])[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------- AllReduce
// Ring layout in the CCL half: [staging ring][result ring], each kDepth x n slices x G channels x sub bytes.
template <typename T, int OP, bool EMU, bool NVLS> __device__ void AllReduceBody(KCtx &k, const CollArgs &A)
{
    __shared__ int sFail;
    const int n = k.nranks;
    const uint64_t slice = Up128((A.bytes + n - 1) / n);
    // The channel walks as many sub-chunks as its longest part needs. That is not always its part of the longest slice: a
    // shorter last slice is cut with a smaller stride, which can leave the LAST channel a longer remainder than slice 0 does.
    uint64_t longestPart = 0;
    for (int j = 0; j < n; ++j) {
        const uint64_t l = PartOf(SliceLen(A.bytes, slice, j), gridDim.x, blockIdx.x).len;
        longestPart = l > longestPart ? l : longestPart;
    }
    Geo g = MakeGeo(k, A, longestPart);
    if (threadIdx.x == 0) sFail = 0;
    __syncthreads();
    const uint64_t resBase = g.RingBytes();
    const int warp = threadIdx.x >> 5;
    if (warp < 6) {                                             // ---- stagers
        Role r{(int)threadIdx.x, 192, 1};
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (c >= (uint32_t)kDepth && !Wait(k, r, MOVED, g.base + c - kDepth + 1, &sFail)) break;
            for (int j = 0; j < n; ++j) {
                Part p = PartOf(SliceLen(A.bytes, slice, j), gridDim.x, blockIdx.x);
                Copy(k.Ccl(k.rank) + g.Slot(d, j), (const char *)A.in + (uint64_t)j * slice + p.off + (uint64_t)c * g.sub, SubLen(p.len, g.sub, c), r);
            }
            Signal(k, r, STAGED, g.base + c + 1);
        }
    } else if (warp < 10) {                                     // ---- movers
        Role r{(int)threadIdx.x - 192, 128, 2};
        Part p = PartOf(SliceLen(A.bytes, slice, k.rank), gridDim.x, blockIdx.x);
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (!Wait(k, r, STAGED, g.base + c + 1, &sFail)) break;
            if (c >= (uint32_t)kDepth && !Wait(k, r, DRAINED, g.base + c - kDepth + 1, &sFail)) break;
            const uint64_t len = SubLen(p.len, g.sub, c);
            if constexpr (NVLS) {
                MoveReduceNvls<T, OP>(k.Mc() + g.Slot(d, k.rank), k.Mc() + resBase + g.Slot(d, k.rank), len, r);
            } else {
                const char *src[kMaxRanks];
                char *dst[kMaxRanks];
                for (int q = 0; q < n; ++q) { src[q] = k.Ccl(q) + g.Slot(d, k.rank); dst[q] = k.Ccl(q) + resBase + g.Slot(d, k.rank); }
                MoveReducePlain<T, OP>(src, n, dst, n, len, r);
            }
            Signal(k, r, MOVED, g.base + c + 1);
        }
    } else {                                                    // ---- drainers
        Role r{(int)threadIdx.x - 320, 192, 3};
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (!Wait(k, r, MOVED, g.base + c + 1, &sFail)) break;
            for (int j = 0; j < n; ++j) {
                Part p = PartOf(SliceLen(A.bytes, slice, j), gridDim.x, blockIdx.x);
                Copy((char *)A.out + (uint64_t)j * slice + p.off + (uint64_t)c * g.sub, k.Ccl(k.rank) + resBase + g.Slot(d, j), SubLen(p.len, g.sub, c), r);
            }
            Signal(k, r, DRAINED, g.base + c + 1);
        }
    }
    Finish(k, g);
}

// ---------------------------------------------------------------------------------------------- ReduceScatter
// sendBytes[j] / sendOff[j]: the block destined to rank j (uniform for the plain operator). One staging ring.
template <typename T, int OP, bool EMU, bool NVLS> __device__ void ReduceScatterBody(KCtx &k, const CollArgs &A)
{
    __shared__ int sFail;
    const int n = k.nranks;
    uint64_t longest = 0;                                       // this channel's longest part over all blocks (see AllReduceBody)
    for (int j = 0; j < n; ++j) {
        const uint64_t l = PartOf(A.sendBytes[j], gridDim.x, blockIdx.x).len;
        longest = l > longest ? l : longest;
    }
    Geo g = MakeGeo(k, A, longest);
    if (threadIdx.x == 0) sFail = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    if (warp < 10) {                                            // ---- stagers (n blocks per sub-chunk)
        Role r{(int)threadIdx.x, 320, 1};
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (c >= (uint32_t)kDepth && !Wait(k, r, MOVED, g.base + c - kDepth + 1, &sFail)) break;
            for (int j = 0; j < n; ++j) {
                Part p = PartOf(A.sendBytes[j], gridDim.x, blockIdx.x);
                Copy(k.Ccl(k.rank) + g.Slot(d, j), (const char *)A.in + A.sendOff[j] + p.off + (uint64_t)c * g.sub, SubLen(p.len, g.sub, c), r);
            }
            Signal(k, r, STAGED, g.base + c + 1);
        }
    } else {                                                    // ---- movers: reduce the own block into the user buffer
        Role r{(int)threadIdx.x - 320, 192, 2};
        Part p = PartOf(A.sendBytes[k.rank], gridDim.x, blockIdx.x);
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (!Wait(k, r, STAGED, g.base + c + 1, &sFail)) break;
            const uint64_t len = SubLen(p.len, g.sub, c);
            char *out = (char *)A.out + p.off + (uint64_t)c * g.sub;
            if constexpr (NVLS) {
                MoveReduceNvlsToLocal<T, OP>(k.Mc() + g.Slot(d, k.rank), (T *)out, len, r);
            } else {
                const char *src[kMaxRanks];
                for (int q = 0; q < n; ++q) src[q] = k.Ccl(q) + g.Slot(d, k.rank);
                char *dst[1] = {out};
                MoveReducePlain<T, OP>(src, n, dst, 1, len, r);
            }
            Signal(k, r, MOVED, g.base + c + 1);
        }
    }
    Finish(k, g);
}

// ---------------------------------------------------------------------------------------------- AllGather(V)
// No input staging: the movers read the user buffer and push sub-chunk c into slot (d, rank) of every rank's ring
// (one multimem.st through the switch, or one plain store per peer); the drainers copy all n slots out.
//
// A2A = true turns the same pipeline into AlltoAll: the piece pushed to rank q is block q of the send buffer
// (sendOff[q], sendBytes[q]) instead of one piece for everybody, always with plain peer stores.
template <bool EMU, bool NVLS, bool A2A = false> __device__ void AllGatherBody(KCtx &k, const CollArgs &A)
{
    __shared__ int sFail;
    const int n = k.nranks;
    uint64_t longest = 0;                                       // this channel's longest part over all blocks (see AllReduceBody)
    for (int j = 0; j < n; ++j) {
        const uint64_t l = PartOf(A.recvBytes[j], gridDim.x, blockIdx.x).len;
        longest = l > longest ? l : longest;
    }
    Geo g = MakeGeo(k, A, longest);
    if (threadIdx.x == 0) sFail = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    if (warp < 6) {                                             // ---- movers (push)
        Role r{(int)threadIdx.x, 192, 1};
        Part p = PartOf(A.recvBytes[k.rank], gridDim.x, blockIdx.x);
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (c >= (uint32_t)kDepth && !Wait(k, r, DRAINED, g.base + c - kDepth + 1, &sFail)) break;
            if constexpr (A2A) {
                for (int q = 0; q < n; ++q) {
                    const int dstRank = (k.rank + q) % n;
                    Part ps = PartOf(A.sendBytes[dstRank], gridDim.x, blockIdx.x);
                    Copy(k.Ccl(dstRank) + g.Slot(d, k.rank), (const char *)A.in + A.sendOff[dstRank] + ps.off + (uint64_t)c * g.sub, SubLen(ps.len, g.sub, c), r);
                }
                Signal(k, r, MOVED, g.base + c + 1);
                continue;
            }
            const uint64_t len = SubLen(p.len, g.sub, c);
            const char *src = (const char *)A.in + p.off + (uint64_t)c * g.sub;
            const uint64_t slot = g.Slot(d, k.rank);
            const int align = ((uintptr_t)src & 15u) == 0 ? 16 : ((uintptr_t)src & 3u) == 0 ? 4 : 1;
            auto load16 = [&](uint64_t i) -> uint4 {
                if (align == 16) return ((const uint4 *)src)[i];
                uint4 v;
                if (align == 4) {
                    const uint32_t *w = (const uint32_t *)(src + (i << 4));
                    v.x = w[0]; v.y = w[1]; v.z = w[2]; v.w = w[3];
                } else {
                    char *b = (char *)&v;
                    for (int t = 0; t < 16; ++t) b[t] = src[(i << 4) + t];
                }
                return v;
            };
            const uint64_t nvec = len >> 4;
            if constexpr (NVLS) {
                constexpr int U = 4;
                char *mc = k.Mc() + slot;
                uint64_t i = r.tid;
                const uint64_t stride = (uint64_t)r.nthr * U;
                for (; i + (uint64_t)r.nthr * (U - 1) < nvec; i += stride) {
                    uint4 v[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) v[u] = load16(i + (uint64_t)u * r.nthr);
#pragma unroll
                    for (int u = 0; u < U; ++u) MultimemSt16(mc + ((i + (uint64_t)u * r.nthr) << 4), v[u]);
                }
                for (; i < nvec; i += r.nthr) MultimemSt16(mc + (i << 4), load16(i));
            } else {
                constexpr int U = 8;
                uint64_t i = r.tid;
                const uint64_t stride = (uint64_t)r.nthr * U;
                for (; i + (uint64_t)r.nthr * (U - 1) < nvec; i += stride) {
                    uint4 v[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) v[u] = load16(i + (uint64_t)u * r.nthr);
                    for (int q = 0; q < n; ++q) {
                        uint4 *dst = (uint4 *)(k.Ccl((k.rank + q) % n) + slot);
#pragma unroll
                        for (int u = 0; u < U; ++u) dst[i + (uint64_t)u * r.nthr] = v[u];
                    }
                }
                for (; i < nvec; i += r.nthr) {
                    uint4 v = load16(i);
                    for (int q = 0; q < n; ++q) ((uint4 *)(k.Ccl((k.rank + q) % n) + slot))[i] = v;
                }
            }
            // a tail shorter than 16 bytes: one plain byte store per rank
            for (uint64_t b = (nvec << 4) + r.tid; b < len; b += r.nthr) {
                char v = src[b];
                for (int q = 0; q < n; ++q) (k.Ccl(q) + slot)[b] = v;
            }
            Signal(k, r, MOVED, g.base + c + 1);
        }
    } else {                                                    // ---- drainers
        Role r{(int)threadIdx.x - 192, 320, 2};
        const bool inPlace = !A2A && (const char *)A.in == (const char *)A.out + A.recvOff[k.rank];
        for (uint32_t c = 0; c < g.chunks; ++c) {
            const int d = c % kDepth;
            if (!Wait(k, r, MOVED, g.base + c + 1, &sFail)) break;
            for (int q = 0; q < n; ++q) {
                int j = (k.rank + q) % n;
                if (j == k.rank && inPlace) continue;
                Part p = PartOf(A.recvBytes[j], gridDim.x, blockIdx.x);
                Copy((char *)A.out + A.recvOff[j] + p.off + (uint64_t)c * g.sub, k.Ccl(k.rank) + g.Slot(d, j), SubLen(p.len, g.sub, c), r);
            }
            Signal(k, r, DRAINED, g.base + c + 1);
        }
    }
    Finish(k, g);
}

}  // namespace pipe
