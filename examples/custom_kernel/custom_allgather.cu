// Writing your own communication kernel against the symmetric heap.
//
// HcclCreateOpResCtx hands back a device-resident description of the communicator: every rank's heap as mapped on this
// device, a workspace window reserved for this operator inside every heap, and 64 KB of zero-initialised flag words.
// This sample implements an all-gather with it: each rank stores its block into slot[rank] of EVERY rank's window with
// plain peer stores, publishes a flag with release semantics, waits (bounded) for every peer's flag and copies the
// gathered window out. It is the counterpart of HCCL's custom-operator samples (reference:
// examples/05_custom_ops_allgather/op_kernel/*, examples/04_custom_ops_p2p/op_kernel_aicpu/*), which acquire channels
// and notify resources from the communicator and then launch their own kernel.
//
// On the simulation backend the same protocol runs as host code over the shared-memory heaps.
#include <atomic>
#include "common.h"
#include "hccl/hccl_mc2.h"

__device__ __forceinline__ void StRelease(uint32_t *p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t LdAcquire(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA. status[0] = 1 when a wait ran out (the kernel still returns; nothing hangs).
__global__ void CustomAllGather(const HcclOpResCtx *ctx, const float *in, float *out, uint64_t count, uint32_t epoch, uint64_t waitNs, uint32_t *status)
{
    const uint32_t me = ctx->rank, n = ctx->nranks;
    const uint64_t slotBytes = count * sizeof(float);
    for (uint32_t d = 0; d < n; ++d) {                                   // push my block into everybody's window
        uint32_t r = (me + d) % n;
        float *dst = (float *)((char *)ctx->heap[r] + ctx->workspaceOff + me * slotBytes);
        for (uint64_t i = threadIdx.x; i < count; i += blockDim.x) dst[i] = in[i];
    }
    __syncthreads();                                                     // all stores of the CTA issued ...
    if (threadIdx.x < n) {
        uint32_t r = threadIdx.x;
        StRelease((uint32_t *)((char *)ctx->heap[r] + ctx->flagOff) + me, epoch);     // ... and released to rank r
        const uint32_t *flag = (const uint32_t *)((char *)ctx->heap[me] + ctx->flagOff) + r;
        uint64_t start;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(start));
        while ((int32_t)(LdAcquire(flag) - epoch) < 0) {
            uint64_t now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (now - start > waitNs) { status[0] = 1; break; }
            __nanosleep(100);
        }
    }
    __syncthreads();
    const float *win = (const float *)((char *)ctx->heap[me] + ctx->workspaceOff);
    for (uint64_t i = threadIdx.x; i < count * n; i += blockDim.x) out[i] = win[i];
}

// The same protocol on the host (simulation backend: the heaps are shared memory of this process).
static bool HostAllGather(const HcclOpResCtx *ctx, const float *in, float *out, uint64_t count, uint32_t epoch)
{
    const uint32_t me = ctx->rank, n = ctx->nranks;
    for (uint32_t r = 0; r < n; ++r) memcpy((char *)ctx->heap[r] + ctx->workspaceOff + me * count * sizeof(float), in, count * sizeof(float));
    for (uint32_t r = 0; r < n; ++r)
        reinterpret_cast<std::atomic<uint32_t> *>((char *)ctx->heap[r] + ctx->flagOff)[me].store(epoch, std::memory_order_release);
    for (uint32_t r = 0; r < n; ++r) {
        auto *flag = reinterpret_cast<std::atomic<uint32_t> *>((char *)ctx->heap[me] + ctx->flagOff) + r;
        for (long spins = 0; (int32_t)(flag->load(std::memory_order_acquire) - epoch) < 0; ++spins) {
            if (spins > 2000000000L) return false;
            std::this_thread::yield();
        }
    }
    memcpy(out, (char *)ctx->heap[me] + ctx->workspaceOff, count * n * sizeof(float));
    return true;
}

int main()
{
    return RunRanks([](RankCtx &c) {
        const uint64_t count = 4096;
        void *args = nullptr, *ctxPtr = nullptr;
        HCCLCHECK(HcclKfcAllocOpArgs(&args));
        HCCLCHECK(HcclKfcOpArgsSetSrcDataType(args, HCCL_DATA_TYPE_FP32));
        HCCLCHECK(HcclKfcOpArgsSetDstDataType(args, HCCL_DATA_TYPE_FP32));
        HCCLCHECK(HcclKfcOpArgsSetCount(args, count));
        char cfg[] = "custom_allgather";
        HCCLCHECK(HcclKfcOpArgsSetAlgConfig(args, cfg));
        HCCLCHECK(HcclCreateOpResCtx(c.comm, HCCL_CMD_ALLGATHER, args, &ctxPtr));
        HCCLCHECK(HcclKfcFreeOpArgs(args));
        HCCLCHECK(HcclBarrier(c.comm, c.stream));            // every rank has created (and zeroed) its window before anyone writes
        c.Sync();

        std::vector<float> mine(count, (float)c.rank + 0.25f), all(count * c.size);
        bool ok = true;
        for (uint32_t epoch = 1; epoch <= 2 && ok; ++epoch) {             // twice: the flags are epochs, not booleans
            if (epoch == 2) {
                // the window is reused: nobody may overwrite it before every rank has read the previous round
                HCCLCHECK(HcclBarrier(c.comm, c.stream));
                c.Sync();
                for (auto &v : mine) v += 100.f;
            }
            if (c.cuda) {
                float *din = (float *)c.Alloc(count * 4), *dout = (float *)c.Alloc(count * 4 * c.size);
                uint32_t *status;
                CUDACHECK(cudaMallocHost(&status, 4));
                *status = 0;
                c.Upload(din, mine.data(), count * 4);
                CustomAllGather<<<1, 256, 0, c.stream>>>((const HcclOpResCtx *)ctxPtr, din, dout, count, epoch, 2000000000ull, status);
                CUDACHECK(cudaGetLastError());
                c.Sync();
                ok = *status == 0;
                c.Download(all.data(), dout, count * 4 * c.size);
                c.Free(din);
                c.Free(dout);
                cudaFreeHost(status);
            } else {
                ok = HostAllGather((const HcclOpResCtx *)ctxPtr, mine.data(), all.data(), count, epoch);
            }
            for (uint32_t r = 0; r < c.size && ok; ++r)
                for (uint64_t i = 0; i < count; ++i)
                    if (all[r * count + i] != (float)r + 0.25f + (epoch == 2 ? 100.f : 0.f)) { ok = false; break; }
        }
        return ok;
    });
}
