// Pieces shared by the fused matmul + collective kernels: per-CTA context (rank, op parity), the entry / exit tickets
// that advance the communicator's device-resident op counter and clear this op's counters, remote counter updates,
// bounded counter waits and bulk (TMA, non-multicast) copies used to push activation shards to peers.
//
// Synchronisation scheme of every fused op:
//   * the op counter of the communicator (DevCtrl::opCount) gives the parity `half`; workspaces and counters exist
//     twice and alternate per op, exactly like the CCL scratch of the plain collectives;
//   * producers bump a counter at the consumer rank (red.release.sys) after their data is written; consumers wait for
//     counter >= expected with a deadline;
//   * the last CTA of an op zeroes the counters of its parity. They are next written by op k+2, which a peer can only
//     enter after it has seen this rank take part in op k+1, i.e. after this kernel has ended.
#pragma once
#include "../kernels/primitives.cuh"
#include "gemm_sm100.cuh"

namespace hccl {
namespace mc2 {

struct FusedCtx {
    const DevComm *c;
    int rank, n;
    char *heap;
    DevCtrl *ctrl;
    DevFlags *flags;
    uint32_t half;
    dev::KCtx k;       // for the bounded waits / timeout reports of the collective primitives
};

__device__ __forceinline__ void FusedInit(const GemmParams &p, FusedCtx &x)
{
    __shared__ uint32_t sHalf, sSeq;
    x.c = (const DevComm *)p.comm;
    x.rank = x.c->rank;
    x.n = x.c->nranks;
    x.heap = x.c->heap[x.rank];
    x.ctrl = CtrlOf(x.heap);
    x.flags = FlagsOf(x.heap);
#ifdef HCCL_DEBUG_BOUNDS
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) dev::g_boundsComm = x.c;
#endif
    if (threadIdx.x == 0) {
        uint32_t oc = dev::LdVolatile(&x.ctrl->opCount);
        sHalf = oc & 1u;
        __threadfence();
        uint32_t t = atomicAdd(&x.ctrl->ticket, 1u);
        if (t == gridDim.x - 1) {
            x.ctrl->ticket = 0;
            __threadfence();
            *((volatile uint32_t *)&x.ctrl->opCount) = oc + 1u;
            if (x.c->progress) *((volatile uint32_t *)x.c->progress) = oc + 1u;
        }
        if (blockIdx.x == 0 && x.c->traceOn) dev::TraceEnter(x.ctrl, oc);
        sSeq = oc;
    }
    __syncthreads();
    x.half = sHalf;
    x.k.c = x.c; x.k.rank = x.rank; x.k.nranks = x.n; x.k.heap = x.heap; x.k.ctrl = x.ctrl; x.k.flags = x.flags;
    x.k.half = x.half; x.k.chan = blockIdx.x; x.k.epoch = 0; x.k.syncs = 0; x.k.ok = true; x.k.seq = sSeq; x.k.vGrid = gridDim.x; x.k.vBlock = blockIdx.x; x.k.cclShift = 0;
}

// Last CTA out clears the counters of this parity.
__device__ __forceinline__ void FusedExit(FusedCtx &x)
{
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0 && x.c->traceOn) dev::TraceLeave(x.ctrl, x.k.seq);
    __shared__ uint32_t sLast;
    if (threadIdx.x == 0) {
        __threadfence();
        uint32_t t = atomicAdd(&x.ctrl->gridBar[0], 1u);
        sLast = (t == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (sLast) {
        uint32_t *r = &x.flags->mc2Ready[x.half][0][0];
        for (uint32_t i = threadIdx.x; i < (uint32_t)kMaxRanks * 64; i += blockDim.x) r[i] = 0;
        uint32_t *d = &x.flags->mc2Done[x.half][0][0];
        for (uint32_t i = threadIdx.x; i < (uint32_t)kMaxRanks * 4; i += blockDim.x) d[i] = 0;
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) x.ctrl->gridBar[0] = 0;
    }
}

// Tile order inside one segment of `rows` row blocks x `nBlocks` column blocks: groups of up to 16 row blocks are walked
// column by column, so a wave of CTAs touches few distinct A and B panels and both stay in L2.
__device__ __forceinline__ void SegmentTile(uint32_t rem, uint32_t rows, uint32_t nBlocks, uint32_t *rowBlk, uint32_t *nb, uint32_t group = 16)
{
    const uint32_t g = rows < group ? rows : group;
    const uint32_t perGroup = g * nBlocks;
    const uint32_t grp = rem / perGroup, first = grp * g;
    const uint32_t size = rows - first < g ? rows - first : g;
    const uint32_t in = rem % perGroup;
    *rowBlk = first + in % size;
    *nb = in / size;
}

// counter at a (possibly remote) rank += v, releasing this thread's (and, after a CTA barrier, this CTA's) prior writes
__device__ __forceinline__ void RemoteAddRelease(uint32_t *addr, uint32_t v)
{
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

// Bounded wait for a local counter; sets the kernel's abort word on expiry.
__device__ __forceinline__ bool WaitCounterGe(FusedCtx &x, const uint32_t *ctr, uint32_t target, uint32_t peer, uint32_t phase, volatile uint32_t *abortWord)
{
    bool ok = dev::WaitFlagGe(x.k, ctr, target, peer, phase);
    if (!ok && abortWord) *abortWord = 1;
    return ok;
}

// ---- bulk copies (TMA, untiled, never multicast). Addresses and sizes are multiples of 16 bytes.
__device__ __forceinline__ void BulkLoad(void *smemDst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(SmemAddr(smemDst)), "l"(gsrc), "r"(bytes),
                 "r"(SmemAddr(bar))
                 : "memory");
}
__device__ __forceinline__ void BulkStore(void *gdst, const void *smemSrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(SmemAddr(smemSrc)), "r"(bytes) : "memory");
}
template <int N> __device__ __forceinline__ void BulkWaitRead() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

}  // namespace mc2
}  // namespace hccl
