// Device-side building blocks of the SM / NVLS engine: system-scope flag accesses, bounded waits that report
// instead of hanging, per-channel barriers with device-resident epochs, ping-pong selection of the CCL half,
// vectorised block copies, typed reductions and multimem (NVLS) accessors.
//
// Replaces what HCCL's vector-core kernels get from AivCommBase (reference:
// src/ops/op_common/template/aiv/aiv_communication_base_v2.h:439-446 Record, :495-505 WaitFlag -- an unbounded
// poll there --, :550-571 BarrierAll, :650-713 CpGM2GM with reduce). Every wait here has a deadline taken from
// DevComm::timeoutNs; on expiry the kernel writes a DevStatus record to pinned host memory, raises the abort flag
// in its control block so sibling CTAs stop early, and returns normally: the context stays usable and the host
// surfaces HCCL_E_TIMEOUT.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../core/dev_comm.h"
#include "hccl/hccl_types.h"

namespace hccl {
namespace dev {

#ifdef HCCL_DEBUG_BOUNDS
static __device__ const DevComm *g_boundsComm = nullptr;   // debug flavor: communicator of the running kernel (see HeapRangeOk)
#endif

// ---------------------------------------------------------------------------------------------- flag accessors
__device__ __forceinline__ uint32_t LdAcquireSys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t LdAcquireSys64(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void StReleaseSys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void StReleaseSys64(uint64_t *p, uint64_t v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t LdVolatile(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t GlobalTimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------------- kernel context
struct KCtx {
    const DevComm *c;
    int rank, nranks;
    char *heap;          // own heap
    DevCtrl *ctrl;
    DevFlags *flags;
    uint32_t half;       // CCL half of this op
    uint32_t chan;       // channel = blockIdx.x
    uint32_t epoch;      // channel epoch at kernel entry; sync point i uses epoch + i
    uint32_t syncs;      // sync points consumed so far
    bool ok;             // false after a timeout
    uint32_t seq;        // op counter value this kernel entered with (trace slot)
    // Work split of the kernel bodies: CTA vBlock of vGrid, scratch offsets shifted by cclShift. The whole grid by default;
    // a kernel that runs two algorithms side by side gives each its own sub-grid and scratch region.
    uint32_t vGrid, vBlock;
    uint64_t cclShift;
    __device__ __forceinline__ char *PeerHeap(int r) const { return c->heap[r]; }
    __device__ __forceinline__ char *Ccl(int r) const { return c->heap[r] + c->cclOff[half] + cclShift; }
    __device__ __forceinline__ char *Mc() const { return c->mcHeap + c->cclOff[half] + cclShift; }
};

__device__ __forceinline__ void ReportTimeout(const KCtx &k, uint32_t peer, uint32_t phase, uint32_t observed, uint32_t expected)
{
    if (atomicCAS(&k.ctrl->abortFlag, 0u, 1u) == 0u) {
        DevStatus *s = k.c->status;
        s->rank = (uint32_t)k.rank;
        s->peer = peer;
        s->channel = k.chan;
        s->phase = phase;
        s->opSeq = k.ctrl->opCount;
        s->observed = observed;
        s->expected = expected;
        __threadfence_system();
        *((volatile uint32_t *)&s->code) = 1u;
        __threadfence_system();
    }
}

// Spins until *flag >= target (wrap-safe). Returns false on timeout or when a sibling CTA already aborted.
__device__ __forceinline__ bool WaitFlagGe(const KCtx &k, const uint32_t *flag, uint32_t target, uint32_t peer, uint32_t phase)
{
    uint64_t start = 0;
    uint32_t spins = 0;
    while (true) {
        uint32_t v = LdAcquireSys(flag);
        if ((int32_t)(v - target) >= 0) return true;
        if ((++spins & 0xffu) == 0) {
            uint64_t now = GlobalTimerNs();
            if (start == 0) start = now;
            if (LdVolatile(&k.ctrl->abortFlag) != 0u) return false;
            if (now - start > k.c->timeoutNs) { ReportTimeout(k, peer, phase, v, target); return false; }
            __nanosleep(64);
        }
    }
}
__device__ __forceinline__ bool WaitFlagGe64(const KCtx &k, const uint64_t *flag, uint64_t target, uint32_t peer, uint32_t phase)
{
    uint64_t start = 0;
    uint32_t spins = 0;
    while (true) {
        uint64_t v = LdAcquireSys64(flag);
        if (v >= target) return true;
        if ((++spins & 0xffu) == 0) {
            uint64_t now = GlobalTimerNs();
            if (start == 0) start = now;
            if (LdVolatile(&k.ctrl->abortFlag) != 0u) return false;
            if (now - start > k.c->timeoutNs) { ReportTimeout(k, peer, phase, (uint32_t)v, (uint32_t)target); return false; }
            __nanosleep(64);
        }
    }
}

// ---- device-side trace (CTA 0, thread 0 only). The record of a kernel is the ring slot of the op counter it entered with;
// the counter has already advanced when later hooks run, so they find their slot through `seq` kept in shared memory.
__device__ __forceinline__ void TraceEnter(DevCtrl *ctrl, uint32_t oc)
{
    DevTraceRec &r = ctrl->trace[oc % kTraceSlots];
    r.seq = oc; r.barriers = 0; r.tBarrier[0] = 0; r.tBarrier[1] = 0; r.tLeave = 0;
    r.tEnter = GlobalTimerNs();
}
__device__ __forceinline__ void TraceBarrier(DevCtrl *ctrl, uint32_t oc)
{
    DevTraceRec &r = ctrl->trace[oc % kTraceSlots];
    if (r.seq != oc) return;
    uint64_t now = GlobalTimerNs();
    if (r.barriers == 0) r.tBarrier[0] = now;
    r.tBarrier[1] = now;
    r.barriers++;
}
__device__ __forceinline__ void TraceLeave(DevCtrl *ctrl, uint32_t oc)
{
    DevTraceRec &r = ctrl->trace[oc % kTraceSlots];
    if (r.seq == oc) r.tLeave = GlobalTimerNs();
}

// Entry protocol of every collective kernel. EMU: several ranks share this GPU and blockIdx.y names the rank.
// Reads the op counter (parity = CCL half) and the channel epoch, then takes a ticket; the last CTA to arrive
// advances the op counter for the next launch.
template <bool EMU> __device__ __forceinline__ KCtx EnterCollective(const DevComm *comms)
{
    __shared__ uint32_t sHalf, sEpoch, sSeq;
    KCtx k;
    k.c = EMU ? &comms[blockIdx.y] : comms;
#ifdef HCCL_DEBUG_BOUNDS
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) g_boundsComm = k.c;
#endif
    k.rank = k.c->rank;
    k.nranks = k.c->nranks;
    k.heap = k.c->heap[k.rank];
    k.ctrl = CtrlOf(k.heap);
    k.flags = FlagsOf(k.heap);
    k.chan = blockIdx.x;
    if (threadIdx.x == 0) {
        uint32_t oc = LdVolatile(&k.ctrl->opCount);
        sHalf = oc & 1u;
        sSeq = oc;
        sEpoch = LdVolatile(&k.ctrl->chanEpoch[k.chan]);
        __threadfence();
        uint32_t t = atomicAdd(&k.ctrl->ticket, 1u);
        if (t == gridDim.x - 1) {
            k.ctrl->ticket = 0;
            __threadfence();
            *((volatile uint32_t *)&k.ctrl->opCount) = oc + 1u;
            if (k.c->progress) *((volatile uint32_t *)k.c->progress) = oc + 1u;
        }
        if (blockIdx.x == 0 && k.c->traceOn) TraceEnter(k.ctrl, oc);
    }
    __syncthreads();
    k.half = sHalf;
    k.epoch = sEpoch;
    k.syncs = 0;
    k.ok = true;
    k.seq = sSeq;
    k.vGrid = gridDim.x; k.vBlock = blockIdx.x; k.cclShift = 0;
    return k;
}

__device__ __forceinline__ void LeaveCollective(KCtx &k)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        *((volatile uint32_t *)&k.ctrl->chanEpoch[k.chan]) = k.epoch + k.syncs;
        if (k.chan == 0 && k.c->traceOn && k.ok) TraceLeave(k.ctrl, k.seq);
    }
}

// Channel barrier across all ranks: every rank's CTA `chan` signals every peer and waits for every peer.
// All stores issued by this CTA before the call are visible to a peer's CTA after its matching call returns.
__device__ __forceinline__ bool ChannelBarrier(KCtx &k, uint32_t phase)
{
    k.syncs++;
    uint32_t target = k.epoch + k.syncs;
    __syncthreads();
    bool mine = true;
    int t = (int)threadIdx.x;
    if (t < k.nranks && t != k.rank) {
        StReleaseSys(&FlagsOf(k.PeerHeap(t))->barrier[k.chan][k.rank], target);
        mine = WaitFlagGe(k, &k.flags->barrier[k.chan][t], target, (uint32_t)t, phase);
    }
    int all = __syncthreads_and(mine ? 1 : 0);
    if (!all) k.ok = false;
    else if (k.chan == 0 && threadIdx.x == 0 && k.c->traceOn) TraceBarrier(k.ctrl, k.seq);
    return all != 0;
}

// One-directional variants for rooted operators.
__device__ __forceinline__ void ChannelSignal(KCtx &k, int peer, uint32_t value)
{
    StReleaseSys(&FlagsOf(k.PeerHeap(peer))->barrier[k.chan][k.rank], value);
}

// ---------------------------------------------------------------------------------------------- partitioning
// Part `b` of `total` bytes split over `parts` CTAs in 128-byte aligned pieces.
struct Part { uint64_t off, len; };
__device__ __forceinline__ Part PartOf(uint64_t total, uint32_t parts, uint32_t b)
{
    uint64_t per = ((total + parts - 1) / parts + 127) & ~127ull;
    uint64_t off = per * b;
    Part p;
    p.off = off < total ? off : total;
    p.len = off < total ? (total - off < per ? total - off : per) : 0;
    return p;
}

// Part `b` of round `t` of a transfer of `total` bytes that moves through a slot of `slot` bytes per round. The split is
// fixed by the first (longest) round, so a CTA touches the same byte range of the slot in every round and the per-CTA
// barriers order its reuse.
__device__ __forceinline__ Part PartOfRound(uint64_t total, uint64_t slot, uint64_t t, uint32_t parts, uint32_t b)
{
    const uint64_t first = total < slot ? total : slot;
    const uint64_t per = ((first + parts - 1) / parts + 127) & ~127ull;
    const uint64_t len = total <= t * slot ? 0 : (total - t * slot < slot ? total - t * slot : slot);
    const uint64_t off = per * b;
    Part p;
    p.off = off < len ? off : len;
    p.len = off < len ? (len - off < per ? len - off : per) : 0;
    return p;
}

// ---------------------------------------------------------------------------------------------- copies
template <int UNROLL> __device__ __forceinline__ void CopyVec16(uint4 *__restrict__ d, const uint4 *__restrict__ s, uint64_t nvec)
{
    const uint64_t stride = (uint64_t)blockDim.x * UNROLL;
    uint64_t i = threadIdx.x;
    for (; i + (uint64_t)blockDim.x * (UNROLL - 1) < nvec; i += stride) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) v[u] = s[i + (uint64_t)u * blockDim.x];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) d[i + (uint64_t)u * blockDim.x] = v[u];
    }
    for (; i < nvec; i += blockDim.x) d[i] = s[i];
}

#ifdef HCCL_DEBUG_BOUNDS
// Debug flavor (-DHCCL_DEBUG_BOUNDS): every kernel registers its communicator at entry; a copy whose source or
// destination starts inside some rank's heap must also end inside it. A violation records status code 2 with the
// offending offset and the copy is skipped -- nothing out of range is ever touched.
__device__ __forceinline__ bool HeapRangeOk(const void *p, uint64_t n)
{
    const DevComm *c = g_boundsComm;
    if (!c) return true;
    const char *b = (const char *)p;
    for (int r = 0; r < c->nranks; ++r) {
        const char *h = c->heap[r];
        if (b >= h && b < h + c->heapBytes) {
            if (b + n <= h + c->heapBytes) return true;
            DevStatus *s = c->status;
            s->rank = (uint32_t)c->rank; s->peer = (uint32_t)r; s->phase = 900; s->observed = (uint32_t)((b - h) >> 10); s->expected = (uint32_t)(c->heapBytes >> 10);
            __threadfence_system();
            *((volatile uint32_t *)&s->code) = 2u;
            return false;
        }
    }
    return true;    // user memory: extent unknown to the library
}
// the same rule for an address inside the multicast mapping of all heaps
__device__ __forceinline__ bool McRangeOk(const void *p, uint64_t n)
{
    const DevComm *c = g_boundsComm;
    if (!c || !c->mcHeap) return true;
    const char *b = (const char *)p;
    if (b < c->mcHeap || b >= c->mcHeap + c->heapBytes) return true;
    if (b + n <= c->mcHeap + c->heapBytes) return true;
    DevStatus *s = c->status;
    s->rank = (uint32_t)c->rank; s->peer = 0xffu; s->phase = 901; s->observed = (uint32_t)((b - c->mcHeap) >> 10); s->expected = (uint32_t)(c->heapBytes >> 10);
    __threadfence_system();
    *((volatile uint32_t *)&s->code) = 2u;
    return false;
}
#define HCCL_CHECK_RANGE(dst, src, n) if (!::hccl::dev::HeapRangeOk(dst, n) || !::hccl::dev::HeapRangeOk(src, n)) return
#define HCCL_RANGE_OK(p, n) (::hccl::dev::HeapRangeOk(p, n) && ::hccl::dev::McRangeOk(p, n))
#else
#define HCCL_CHECK_RANGE(dst, src, n)
#define HCCL_RANGE_OK(p, n) true
#endif

// Copies `n` bytes with all threads of the CTA. Any alignment; 16-byte vectors when both sides allow it.
__device__ __forceinline__ void BlockCopy(void *dst, const void *src, uint64_t n)
{
    if (n == 0) return;
    HCCL_CHECK_RANGE(dst, src, n);
    uintptr_t a = (uintptr_t)dst | (uintptr_t)src;
    if ((a & 15u) == 0) {
        uint64_t nvec = n >> 4;
        CopyVec16<4>((uint4 *)dst, (const uint4 *)src, nvec);
        uint64_t done = nvec << 4;
        for (uint64_t i = done + threadIdx.x; i < n; i += blockDim.x) ((char *)dst)[i] = ((const char *)src)[i];
    } else if ((a & 3u) == 0) {
        uint64_t nw = n >> 2;
        for (uint64_t i = threadIdx.x; i < nw; i += blockDim.x) ((uint32_t *)dst)[i] = ((const uint32_t *)src)[i];
        for (uint64_t i = (nw << 2) + threadIdx.x; i < n; i += blockDim.x) ((char *)dst)[i] = ((const char *)src)[i];
    } else {
        for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) ((char *)dst)[i] = ((const char *)src)[i];
    }
}

// ---------------------------------------------------------------------------------------------- typed reduction
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type ToAcc(T v) { return v; }
template <> __device__ __forceinline__ float ToAcc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ToAcc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T FromAcc(typename Acc<T>::type v) { return v; }
template <> __device__ __forceinline__ __half FromAcc<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 FromAcc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <int OP, typename A> __device__ __forceinline__ A Combine(A a, A b)
{
    if (OP == HCCL_REDUCE_SUM) return a + b;
    if (OP == HCCL_REDUCE_PROD) return a * b;
    if (OP == HCCL_REDUCE_MAX) return a > b ? a : b;
    return a < b ? a : b;
}

// out[i] = slot_0[i] (op) slot_1[i] ... (op) slot_{n-1}[i], slots in rank order (the same order on every rank, so
// every rank that reduces the same data obtains identical bits). Half-precision types accumulate in fp32.
// slot r lives at slotBase[r] (local or peer memory), all 16-byte aligned. `out2` optionally receives a second copy.
template <typename T, int OP, int MAXR>
__device__ __forceinline__ void ReduceSlots(T *out, T *out2, const char *const *slotBase, int nslots, uint64_t nElems)
{
    using A = typename Acc<T>::type;
    constexpr int VE = 16 / sizeof(T);
    for (int r = 0; r < nslots; ++r) if (!HCCL_RANGE_OK(slotBase[r], nElems * sizeof(T))) return;
    if (!HCCL_RANGE_OK(out, nElems * sizeof(T)) || (out2 && !HCCL_RANGE_OK(out2, nElems * sizeof(T)))) return;
    bool vecOk = (((uintptr_t)out | (uintptr_t)out2) & 15u) == 0;
    uint64_t nvec = vecOk ? nElems / VE : 0;
    for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
        A acc[VE];
        {
            uint4 raw = ((const uint4 *)slotBase[0])[i];
            const T *e = (const T *)&raw;
#pragma unroll
            for (int j = 0; j < VE; ++j) acc[j] = ToAcc<T>(e[j]);
        }
        for (int r = 1; r < nslots; ++r) {
            uint4 raw = ((const uint4 *)slotBase[r])[i];
            const T *e = (const T *)&raw;
#pragma unroll
            for (int j = 0; j < VE; ++j) acc[j] = Combine<OP, A>(acc[j], ToAcc<T>(e[j]));
        }
        uint4 res;
        T *e = (T *)&res;
#pragma unroll
        for (int j = 0; j < VE; ++j) e[j] = FromAcc<T>(acc[j]);
        ((uint4 *)out)[i] = res;
        if (out2) ((uint4 *)out2)[i] = res;
    }
    for (uint64_t i = nvec * VE + threadIdx.x; i < nElems; i += blockDim.x) {
        A acc = ToAcc<T>(((const T *)slotBase[0])[i]);
        for (int r = 1; r < nslots; ++r) acc = Combine<OP, A>(acc, ToAcc<T>(((const T *)slotBase[r])[i]));
        T v = FromAcc<T>(acc);
        out[i] = v;
        if (out2) out2[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------- multimem (NVLS)
// 16-byte reduce-load from the multicast address: the switch returns the element-wise reduction over all ranks.
template <typename T, int OP> struct MultimemLdReduce;
template <> struct MultimemLdReduce<float, HCCL_REDUCE_SUM> {
    __device__ __forceinline__ static uint4 Ld(const void *mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
#define HCCL_MM_HALF(T, PTXT, OPV, OPNAME, ACC)                                                                                    \
    template <> struct MultimemLdReduce<T, OPV> {                                                                                  \
        __device__ __forceinline__ static uint4 Ld(const void *mc)                                                                 \
        {                                                                                                                          \
            uint4 v;                                                                                                               \
            asm volatile("multimem.ld_reduce.relaxed.sys.global." OPNAME ACC ".v4." PTXT " {%0,%1,%2,%3}, [%4];"                   \
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                                       \
            return v;                                                                                                              \
        }                                                                                                                          \
    };
HCCL_MM_HALF(__nv_bfloat16, "bf16x2", HCCL_REDUCE_SUM, "add", ".acc::f32")
HCCL_MM_HALF(__nv_bfloat16, "bf16x2", HCCL_REDUCE_MAX, "max", "")
HCCL_MM_HALF(__nv_bfloat16, "bf16x2", HCCL_REDUCE_MIN, "min", "")
HCCL_MM_HALF(__half, "f16x2", HCCL_REDUCE_SUM, "add", ".acc::f32")
HCCL_MM_HALF(__half, "f16x2", HCCL_REDUCE_MAX, "max", "")
HCCL_MM_HALF(__half, "f16x2", HCCL_REDUCE_MIN, "min", "")
#undef HCCL_MM_HALF

__device__ __forceinline__ void MultimemSt16(void *mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

}  // namespace dev
}  // namespace hccl
