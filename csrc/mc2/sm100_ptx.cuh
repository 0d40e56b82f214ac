// Inline-PTX wrappers for the Blackwell (sm_100a) data path used by the fused GEMM kernels: mbarrier, TMA tiled
// loads (never cluster-multicast), tcgen05 tensor-memory allocation, UMMA issue / commit, TMEM loads, and the
// shared-memory / instruction descriptors that tcgen05.mma consumes.
//
// Descriptor bit layouts (checked against the public CUTLASS definitions of UMMA::SmemDescriptor and
// UMMA::InstrDescriptor):
//   smem descriptor (64 bit): [0,14) start address >> 4 | [16,30) leading byte offset >> 4 | [32,46) stride byte
//     offset >> 4 | [46,48) version = 1 | [49,52) base offset | [61,64) layout (2 = 128-byte swizzle)
//   instruction descriptor (32 bit): [4,6) D format (1 = f32) | [7,10) A format | [10,13) B format (1 = bf16,
//     0 = f16 / e4m3) | [15] A major | [16] B major (0 = K-major) | [17,23) N >> 3 | [24,29) M >> 4
//   (the block-scaled form used by the MXFP8 kernels is described at MakeInstrDescMx)
// Every wait is bounded: after the limit the caller gets `false`, raises the kernel's error word and unwinds
// (the TMEM allocation is released before the CTA exits).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hccl {
namespace sm100 {

__device__ __forceinline__ uint32_t SmemAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool ElectOne()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void MbarInit(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarInitFence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void MbarExpectTx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait with a suspend-time hint: the hardware may keep the thread parked up to `hintNs` before it reports "not yet",
// so a long wait costs a handful of instructions instead of a polling loop that occupies an issue slot.
__device__ __forceinline__ bool MbarTryWaitHint(uint64_t *bar, uint32_t parity, uint32_t hintNs)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity), "r"(hintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait built on it (hintNs = 0 falls back to the plain polling wait). sleepNs > 0 adds a nanosleep between polls:
// only for waits that are off the critical path.
__device__ __forceinline__ bool MbarWaitHint(uint64_t *bar, uint32_t parity, volatile uint32_t *abortWord, uint32_t hintNs, uint32_t sleepNs = 0)
{
    uint64_t start = 0;
    uint32_t spins = 0;
    while (!(hintNs ? MbarTryWaitHint(bar, parity, hintNs) : MbarTryWait(bar, parity))) {
        if (sleepNs) __nanosleep(sleepNs);
        if ((++spins & (hintNs || sleepNs ? 0xfu : 0x3ffu)) == 0) {
            uint64_t now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            if (*abortWord != 0 || now - start > 2000000000ull) { *abortWord = 1; return false; }
        }
    }
    return true;
}

// Bounded wait: ~2 s of polling at most; false => the caller must unwind.
__device__ __forceinline__ bool MbarWait(uint64_t *bar, uint32_t parity, volatile uint32_t *abortWord)
{
    uint64_t start = 0;
    uint32_t spins = 0;
    while (!MbarTryWait(bar, parity)) {
        if ((++spins & 0x3ffu) == 0) {
            uint64_t now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            if (*abortWord != 0 || now - start > 2000000000ull) { *abortWord = 1; return false; }
        }
    }
    return true;
}

// Same wait for threads that are off the critical path (epilogue warps waiting for a whole tile, the producer waiting for a
// free stage): between polls the thread sleeps `sleepNs`, so a 128-thread group does not burn issue slots (and power
// under the board's cap) for the tens of microseconds a main loop takes.
__device__ __forceinline__ bool MbarWaitRelaxed(uint64_t *bar, uint32_t parity, volatile uint32_t *abortWord, uint32_t sleepNs)
{
    uint64_t start = 0;
    uint32_t spins = 0;
    while (!MbarTryWait(bar, parity)) {
        if (sleepNs) __nanosleep(sleepNs);
        if ((++spins & 0xffu) == 0) {
            uint64_t now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            if (*abortWord != 0 || now - start > 2000000000ull) { *abortWord = 1; return false; }
        }
    }
    return true;
}

// ---------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void PrefetchTmap(const CUtensorMap *m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// 2-D tiled load global -> shared, completion on an mbarrier of this CTA. x = innermost coordinate (must keep
// x * elemSize a multiple of 16 bytes), y = row.
__device__ __forceinline__ void TmaLoad2D(void *smemDst, const CUtensorMap *m, uint64_t *bar, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(SmemAddr(smemDst)),
                 "l"(m), "r"(SmemAddr(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void TmaStore2D(const CUtensorMap *m, const void *smemSrc, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(m), "r"(SmemAddr(smemSrc)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void TmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void TmaStoreWaitRead0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void TmaStoreWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsyncGlobal() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- tensor memory
__device__ __forceinline__ void TmemAlloc(uint32_t *smemOut, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemOut)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread. accumulate = 0 overwrites D.
__device__ __forceinline__ void UmmaF16(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Block-scaled fp8 (MXFP8): e4m3 operands, one e8m0 scale per 1 x 32 block of K for every row of A and of B, fp32
// accumulate. One instruction covers K = 32; the scales sit in tensor memory (`sfaTmem`, `sfbTmem`: 32-bit columns that
// hold the scales of four consecutive K blocks, the instruction descriptor's scale-factor ids select the byte).
__device__ __forceinline__ void UmmaMxf8(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t sfaTmem, uint32_t sfbTmem,
                                         uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(dTmem),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(sfaTmem), "r"(sfbTmem)
        : "memory");
}
// Shared memory -> tensor memory copy of one scale-factor atom: 32 rows x 16 bytes (512 contiguous bytes) land in 4
// consecutive TMEM columns of lanes 0..31 and are replicated into the other three 32-lane quarters. Issued by one
// thread; ordered with the tcgen05.mma instructions the same thread issues afterwards.
__device__ __forceinline__ void TmemCpSfAtom(uint32_t dstTmem, uint64_t smemDesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dstTmem), "l"(smemDesc) : "memory");
}
// Descriptor of such an atom: no swizzle, rows 16 bytes apart, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t MakeSfSmemDesc(uint32_t smemAddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smemAddr >> 4) & 0x3fffu);
    d |= (uint64_t)(128 >> 4) << 32;        // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version (Blackwell)
    return d;                               // layout type 0 = no swizzle
}
// Untiled bulk copy global -> shared (never multicast); addresses and size are multiples of 16 bytes.
__device__ __forceinline__ void BulkLoadG2S(void *smemDst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(SmemAddr(smemDst)), "l"(gsrc), "r"(bytes),
                 "r"(SmemAddr(bar))
                 : "memory");
}
// Arrives on the mbarrier once all previously issued UMMAs of this thread have completed.
__device__ __forceinline__ void UmmaCommit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (row) base+i.
__device__ __forceinline__ void TmemLd32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- descriptors
// K-major operand tile in shared memory written by a 128-byte-swizzled TMA load: rows of 128 bytes, 8-row swizzle
// atoms of 1024 bytes (so the tile base must be 1024-byte aligned and the stride byte offset is 1024).
__device__ __forceinline__ uint64_t MakeSmemDescSw128(uint32_t smemAddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smemAddr >> 4) & 0x3fffu);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused with swizzled K-major layouts)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// Advance along K inside the swizzle atom by `bytes` (a multiple of 32): only the start-address field moves.
__device__ __forceinline__ uint64_t AdvanceDescK(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }

enum : uint32_t { FMT_F16 = 0, FMT_BF16 = 1, FMT_E4M3 = 0, FMT_E5M2 = 1 };
__host__ __device__ constexpr uint32_t MakeInstrDesc(uint32_t aFmt, uint32_t bFmt, uint32_t m, uint32_t n)
{
    return (1u << 4) | (aFmt << 7) | (bFmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Block-scaled variant (checked against the public CUTLASS definition of UMMA::InstrDescriptorBlockScaled):
//   [4,6) B scale-factor id | [7,10) A format | [10,13) B format (0 = e4m3) | [15] A major | [16] B major | [17,23) N >> 3 |
//   [23] scale format (1 = e8m0) | [24,29) M >> 4 | [29,31) A scale-factor id. The accumulator is always fp32.
__host__ __device__ constexpr uint32_t MakeInstrDescMx(uint32_t m, uint32_t n, uint32_t sfId)
{
    return (sfId << 4) | (FMT_E4M3 << 7) | (FMT_E4M3 << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sfId << 29);
}

}  // namespace sm100
}  // namespace hccl
