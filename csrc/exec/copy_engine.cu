// Copy-engine executor (see copy_engine.h): schedule IR on a CUDA communicator with host-issued work only.
//   LOCAL_COPY / WRITE / READ      cudaMemcpyAsync between (peer-mapped) device addresses -> DMA engines, no SM time
//   *_REDUCE                       one small typed kernel: dst = dst (op) src, src or dst may be peer memory
//   POST / WAIT                    one-thread kernels on counting notify words in the heap; WAIT is bounded
// Queue 0 runs on the caller's stream, further queues (BatchSendRecv) on helper streams forked / joined with events.
// Every plan is bracketed by a notify barrier so that this engine can be mixed freely with the SM / NVLS kernels, whose
// scratch-half parity lives on the device.
#include "../common/launch_count.h"
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include "../common/dtype.h"
#include "../common/log.h"
#include "../kernels/primitives.cuh"
#include "copy_engine.h"

namespace hccl {
namespace {

using namespace dev;

__global__ void PostKernel(const DevComm *c, uint32_t peer, uint32_t slot)
{
    char *heap = c->heap[c->rank];
    DevCtrl *ctrl = CtrlOf(heap);
    uint64_t v = ++ctrl->hostNotifySent[peer][slot];
    __threadfence_system();
    StReleaseSys64(&FlagsOf(c->heap[peer])->hostNotify[c->rank][slot], v);
}

__global__ void WaitKernel(const DevComm *c, uint32_t peer, uint32_t slot)
{
    KCtx k;
    k.c = c; k.rank = c->rank; k.nranks = c->nranks; k.heap = c->heap[c->rank];
    k.ctrl = CtrlOf(k.heap); k.flags = FlagsOf(k.heap); k.chan = 0; k.half = 0; k.epoch = 0; k.syncs = 0; k.ok = true;
    uint64_t want = k.ctrl->hostNotifyWaited[peer][slot] + 1;
    if (WaitFlagGe64(k, &k.flags->hostNotify[peer][slot], want, peer, 100 + slot)) k.ctrl->hostNotifyWaited[peer][slot] = want;
}

template <typename T, int OP> __global__ void ReduceKernel(T *dst, const T *src, uint64_t n)
{
    using A = typename Acc<T>::type;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = FromAcc<T>(Combine<OP, A>(ToAcc<T>(dst[i]), ToAcc<T>(src[i])));
}

template <typename T> cudaError_t LaunchReduceT(void *dst, const void *src, uint64_t n, HcclReduceOp op, cudaStream_t s)
{
    int grid = (int)std::min<uint64_t>((n + 255) / 256, 592);
    switch (op) {
        case HCCL_REDUCE_SUM: ReduceKernel<T, HCCL_REDUCE_SUM><<<grid, 256, 0, s>>>((T *)dst, (const T *)src, n); break;
        case HCCL_REDUCE_PROD: ReduceKernel<T, HCCL_REDUCE_PROD><<<grid, 256, 0, s>>>((T *)dst, (const T *)src, n); break;
        case HCCL_REDUCE_MAX: ReduceKernel<T, HCCL_REDUCE_MAX><<<grid, 256, 0, s>>>((T *)dst, (const T *)src, n); break;
        default: ReduceKernel<T, HCCL_REDUCE_MIN><<<grid, 256, 0, s>>>((T *)dst, (const T *)src, n); break;
    }
    return cudaGetLastError();
}

cudaError_t LaunchReduce(void *dst, const void *src, uint64_t bytes, HcclDataType dt, HcclReduceOp op, cudaStream_t s)
{
    uint64_t n = bytes / DataTypeSize(dt);
    switch (dt) {
        case HCCL_DATA_TYPE_INT8: return LaunchReduceT<int8_t>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_INT16: return LaunchReduceT<int16_t>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_INT32: return LaunchReduceT<int32_t>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_INT64: return LaunchReduceT<long long>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_UINT64: return LaunchReduceT<unsigned long long>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_UINT8: return LaunchReduceT<uint8_t>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_UINT16: return LaunchReduceT<uint16_t>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_UINT32: return LaunchReduceT<uint32_t>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_FP16: return LaunchReduceT<__half>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_FP32: return LaunchReduceT<float>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_FP64: return LaunchReduceT<double>(dst, src, n, op, s);
        case HCCL_DATA_TYPE_BFP16: return LaunchReduceT<__nv_bfloat16>(dst, src, n, op, s);
        default: return cudaErrorInvalidValue;
    }
}

std::mutex g_mu;

constexpr uint32_t kSlotPlanBarrier = kNotifySlots - 1;

}  // namespace

HcclResult CopyEngineRun(Comm *c, const Plan &plan, const ExecBuffers &bufs, cudaStream_t stream, bool isCollective)
{
    const DevComm &d = c->devComm;
    auto local = [&](const BufRef &b) -> char * {
        switch (b.kind) {
            case BufKind::INPUT: return bufs.in + b.off;
            case BufKind::OUTPUT: return bufs.out + b.off;
            case BufKind::CCL: return c->heap[c->rank] + d.cclOff[bufs.cclHalf] + b.off;
            case BufKind::MAILBOX: return c->heap[c->rank] + d.mailboxOff + b.off;
            case BufKind::ABS: return reinterpret_cast<char *>(b.off);
        }
        return nullptr;
    };
    auto remote = [&](uint32_t rank, const BufRef &b) -> char * {
        return c->heap[rank] + (b.kind == BufKind::MAILBOX ? d.mailboxOff : d.cclOff[bufs.cclHalf]) + b.off;
    };
    auto barrier = [&](cudaStream_t s) {
        for (uint32_t k = 1; k < c->nranks; ++k) PostKernel<<<1, 1, 0, s>>>(c->devCommPtr, (c->rank + k) % c->nranks, kSlotPlanBarrier);
        for (uint32_t k = 1; k < c->nranks; ++k) WaitKernel<<<1, 1, 0, s>>>(c->devCommPtr, (c->rank + k) % c->nranks, kSlotPlanBarrier);
    };
    std::lock_guard<std::mutex> lk(g_mu);
    const size_t nq = plan.queues.size();
    if (nq > 1 || !isCollective) {
        HCCL_ERROR("copy engine: %s need launches that wait on one another on one GPU; use the SM engine",
                   isCollective ? "schedules with several queues" : "point-to-point schedules");
        return HCCL_E_NOT_SUPPORT;
    }
    barrier(stream);
    for (size_t q = 0; q < nq; ++q) {
        cudaStream_t s = stream;
        for (const Task &t : plan.queues[q]) {
            cudaError_t e = cudaSuccess;
            switch (t.type) {
                case TaskType::LOCAL_COPY:
                    if (local(t.dst) != local(t.src)) e = cudaMemcpyAsync(local(t.dst), local(t.src), t.bytes, cudaMemcpyDeviceToDevice, s);
                    break;
                case TaskType::WRITE: e = cudaMemcpyAsync(remote(t.rank, t.dst), local(t.src), t.bytes, cudaMemcpyDeviceToDevice, s); break;
                case TaskType::READ: e = cudaMemcpyAsync(local(t.dst), remote(t.rank, t.src), t.bytes, cudaMemcpyDeviceToDevice, s); break;
                case TaskType::LOCAL_REDUCE: e = LaunchReduce(local(t.dst), local(t.src), t.bytes, plan.dtype, plan.op, s); break;
                case TaskType::WRITE_REDUCE: e = LaunchReduce(remote(t.rank, t.dst), local(t.src), t.bytes, plan.dtype, plan.op, s); break;
                case TaskType::READ_REDUCE: e = LaunchReduce(local(t.dst), remote(t.rank, t.src), t.bytes, plan.dtype, plan.op, s); break;
                case TaskType::POST: PostKernel<<<1, 1, 0, s>>>(c->devCommPtr, t.rank, t.slot); e = cudaGetLastError(); break;
                case TaskType::WAIT: WaitKernel<<<1, 1, 0, s>>>(c->devCommPtr, t.rank, t.slot); e = cudaGetLastError(); break;
                default: HCCL_ERROR("copy engine: task type %s is not supported", TaskTypeName(t.type)); return HCCL_E_NOT_SUPPORT;
            }
            if (e != cudaSuccess) { HCCL_ERROR("copy engine: %s failed: %s", TaskTypeName(t.type), cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
            c->counters.kernelsLaunched++;
            CountLaunch();
        }
    }
    barrier(stream);
    return HCCL_SUCCESS;
}

}  // namespace hccl
