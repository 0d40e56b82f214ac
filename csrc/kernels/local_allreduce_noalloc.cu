// All-reduce across buffers of one GPU with the scratch in a file-scope device array: the entry point for callers that
// cannot allocate (see include/hccl/hccl_noalloc.h). No counterpart in HCCL.
//
// Layout of the scratch array:
//   [0, 4 KiB)        DevComm[4]      one description per emulated rank
//   [4 KiB, 12 KiB)   CollArgs[4]     per-call argument blocks
//   [12 KiB, 16 KiB)  DevStatus[4]    where a kernel would record a wait that ran out
//   [64 KiB, ...)     4 rank heaps of kRankHeapBytes: 256 KiB control block + flags, then two 512 KiB staging halves
// In host code `g_scratch` is only a handle for the runtime, not a device address; the device address comes from
// cudaGetSymbolAddress, once per device, and everything the kernel sees is derived from it.
#include <cuda_runtime.h>
#include <cstring>
#include "../common/dtype.h"
#include "../common/log.h"
#include "../common/param_check.h"
#include "coll_args.h"
#include "hccl/hccl_noalloc.h"

namespace hccl {
HcclResult SmIssueEmuLaunch(const DevComm *devComms, int nranks, const SmLaunch &l0, const CollArgs *devArgs, const BatchArgs *devBatch,
                            cudaStream_t stream, bool pairKernel);
}

namespace {

using namespace hccl;

constexpr uint64_t kHeaderBytes = 256 << 10;                 // control block + flag arena of one rank
constexpr uint64_t kHalfBytes = 512 << 10;                   // one staging half
constexpr uint64_t kRankHeapBytes = kHeaderBytes + 2 * kHalfBytes;
constexpr uint64_t kHeapsOff = 64 << 10;
constexpr uint64_t kCommOff = 0, kArgsOff = 4 << 10, kStatusOff = 12 << 10;
constexpr uint64_t kScratchBytes = kHeapsOff + HCCL_NOALLOC_MAX_BUFFERS * kRankHeapBytes;
static_assert(kCtrlBytes + sizeof(DevFlags) <= kHeaderBytes, "control block and flags must fit the header");
static_assert(sizeof(DevComm) * HCCL_NOALLOC_MAX_BUFFERS <= kArgsOff - kCommOff, "DevComm table too large");
static_assert(sizeof(CollArgs) * HCCL_NOALLOC_MAX_BUFFERS <= kStatusOff - kArgsOff, "argument table too large");

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
char *g_devPtr[kMaxDevices] = {nullptr};    // device address of g_scratch, per device ordinal

// Once per device, with that device current: resolve the device address and write the rank descriptions.
HcclResult SetupDevice(int dev, char **out)
{
    if (g_devPtr[dev] == nullptr) {
        char *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            HCCL_ERROR("HcclLocalAllReduceNoAlloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return HCCL_E_RUNTIME;
        }
        g_devPtr[dev] = ptr;
    }
    *out = g_devPtr[dev];
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" HcclResult HcclLocalAllReduceNoAlloc(const void *const *sendBufs, void *const *recvBufs, uint32_t nBufs, uint64_t count,
                                                HcclDataType dataType, HcclReduceOp op, cudaStream_t stream)
{
    if (!sendBufs || !recvBufs) { HCCL_ERROR("[EI0003] HcclLocalAllReduceNoAlloc: buffer tables are null"); return HCCL_E_PTR; }
    if (nBufs < 2 || nBufs > HCCL_NOALLOC_MAX_BUFFERS) {
        HCCL_ERROR("[EI0003] HcclLocalAllReduceNoAlloc: %u buffers requested, supported range is 2..%d", nBufs, HCCL_NOALLOC_MAX_BUFFERS);
        return HCCL_E_PARA;
    }
    HcclResult r = HcomCheckReduceDataType(dataType, op);
    if (r != HCCL_SUCCESS) return r;
    if (count == 0) return HCCL_SUCCESS;
    const uint64_t bytes = count * DataTypeSize(dataType);
    if (bytes > HCCL_NOALLOC_MAX_BYTES) {
        HCCL_ERROR("[EI0003] HcclLocalAllReduceNoAlloc: %llu bytes per buffer exceed the fixed scratch (maximum %u bytes); use a communicator "
                   "for larger payloads", (unsigned long long)bytes, HCCL_NOALLOC_MAX_BYTES);
        return HCCL_E_PARA;
    }
    for (uint32_t i = 0; i < nBufs; ++i)
        if (!sendBufs[i] || !recvBufs[i]) { HCCL_ERROR("[EI0003] HcclLocalAllReduceNoAlloc: buffer %u is null", i); return HCCL_E_PTR; }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return HCCL_E_RUNTIME;
    char *base = nullptr;
    r = SetupDevice(dev, &base);
    if (r != HCCL_SUCCESS) return r;

    // rank descriptions and per-call arguments (small pageable-to-device copies; the runtime stages them before returning)
    // (plain stack arrays: the host side takes nothing from the heap either)
    DevComm comms[HCCL_NOALLOC_MAX_BUFFERS];
    CollArgs args[HCCL_NOALLOC_MAX_BUFFERS];
    SmLaunch launch;
    memset(&launch, 0, sizeof(launch));
    launch.kernel = K_ALLREDUCE_TWOSHOT;
    launch.dtype = dataType;
    launch.ctas = SmCtasFor(bytes * 2 / nBufs, 4u);
    // the two-shot kernel needs (nBufs + 1) slices of ceil(bytes / nBufs), 128-byte aligned, inside one staging half
    if ((uint64_t)(nBufs + 1) * (((bytes + nBufs - 1) / nBufs + 127) & ~127ull) > kHalfBytes) {
        HCCL_ERROR("HcclLocalAllReduceNoAlloc: payload does not fit the staging half");
        return HCCL_E_INTERNAL;
    }
    for (uint32_t i = 0; i < nBufs; ++i) {
        DevComm &d = comms[i];
        memset(&d, 0, sizeof(d));
        d.rank = (int32_t)i;
        d.nranks = (int32_t)nBufs;
        d.heapBytes = kRankHeapBytes;
        for (uint32_t q = 0; q < nBufs; ++q) d.heap[q] = base + kHeapsOff + q * kRankHeapBytes;
        d.cclOff[0] = kHeaderBytes;
        d.cclOff[1] = kHeaderBytes + kHalfBytes;
        d.cclBytes = kHalfBytes;
        d.timeoutNs = 2000000000ull;
        d.status = reinterpret_cast<DevStatus *>(base + kStatusOff) + i;
        d.emuRanks = (int32_t)nBufs;
        CollArgs &a = args[i];
        memset(&a, 0, sizeof(a));
        a.in = sendBufs[i];
        a.out = recvBufs[i];
        a.count = count;
        a.bytes = bytes;
        a.elemSize = DataTypeSize(dataType);
        a.op = (uint32_t)op;
    }
    launch.args = args[0];
    // everything that must start at zero: control blocks, flags, status words (epochs and parity restart every call)
    for (uint32_t i = 0; i < nBufs; ++i)
        if (cudaMemsetAsync(base + kHeapsOff + i * kRankHeapBytes, 0, kHeaderBytes, stream) != cudaSuccess) return HCCL_E_RUNTIME;
    if (cudaMemsetAsync(base + kStatusOff, 0, sizeof(DevStatus) * HCCL_NOALLOC_MAX_BUFFERS, stream) != cudaSuccess) return HCCL_E_RUNTIME;
    if (cudaMemcpyAsync(base + kCommOff, comms, sizeof(DevComm) * nBufs, cudaMemcpyHostToDevice, stream) != cudaSuccess) return HCCL_E_RUNTIME;
    if (cudaMemcpyAsync(base + kArgsOff, args, sizeof(CollArgs) * nBufs, cudaMemcpyHostToDevice, stream) != cudaSuccess) return HCCL_E_RUNTIME;
    r = SmIssueEmuLaunch(reinterpret_cast<const DevComm *>(base + kCommOff), (int)nBufs, launch, reinterpret_cast<const CollArgs *>(base + kArgsOff),
                         nullptr, stream, false);
    if (r != HCCL_SUCCESS) HCCL_ERROR("HcclLocalAllReduceNoAlloc: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return r;
}
