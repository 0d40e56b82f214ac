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
#include <atomic>
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
// device address of g_scratch, per device ordinal. Host threads may race to fill an entry: every one of them resolves
// the same address, so a relaxed atomic publish is enough.
std::atomic<char *> g_devPtr[kMaxDevices];

// Once per device, with that device current: resolve the device address of the scratch array.
HcclResult SetupDevice(int dev, char **out)
{
    char *ptr = g_devPtr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            HCCL_ERROR("HcclLocalAllReduceNoAlloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return HCCL_E_RUNTIME;
        }
        g_devPtr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return HCCL_SUCCESS;
}

// Everything a call contributes, passed BY VALUE as a kernel parameter: the launch owns its copy, so nothing on the
// host (stack or heap) has to outlive the call.
struct CallTable {
    const void *in[HCCL_NOALLOC_MAX_BUFFERS];
    void *out[HCCL_NOALLOC_MAX_BUFFERS];
    uint64_t count, bytes;
    uint32_t elemSize, op, nBufs, pad;
};

// One small CTA: clears what must start at zero (control blocks, flag arenas, status records; epochs and parity
// restart every call) and writes the rank descriptions and argument blocks into the scratch array.
__global__ void NoAllocSetupKernel(CallTable t)
{
    char *base = reinterpret_cast<char *>(g_scratch);      // device code may name the array directly
    for (uint32_t i = 0; i < t.nBufs; ++i) {
        uint4 *h = reinterpret_cast<uint4 *>(base + kHeapsOff + i * kRankHeapBytes);
        for (uint32_t v = threadIdx.x; v < kHeaderBytes / 16; v += blockDim.x) h[v] = make_uint4(0, 0, 0, 0);
    }
    uint32_t *st = reinterpret_cast<uint32_t *>(base + kStatusOff);
    for (uint32_t v = threadIdx.x; v < sizeof(DevStatus) * HCCL_NOALLOC_MAX_BUFFERS / 4; v += blockDim.x) st[v] = 0;
    uint32_t *tab = reinterpret_cast<uint32_t *>(base + kCommOff);
    for (uint32_t v = threadIdx.x; v < (uint32_t)(kStatusOff - kCommOff) / 4; v += blockDim.x) tab[v] = 0;
    __syncthreads();
    if (threadIdx.x < t.nBufs) {
        const uint32_t i = threadIdx.x;
        DevComm &d = reinterpret_cast<DevComm *>(base + kCommOff)[i];
        d.rank = (int32_t)i;
        d.nranks = (int32_t)t.nBufs;
        d.heapBytes = kRankHeapBytes;
        for (uint32_t q = 0; q < t.nBufs; ++q) d.heap[q] = base + kHeapsOff + q * kRankHeapBytes;
        d.cclOff[0] = kHeaderBytes;
        d.cclOff[1] = kHeaderBytes + kHalfBytes;
        d.cclBytes = kHalfBytes;
        d.timeoutNs = 2000000000ull;
        d.status = reinterpret_cast<DevStatus *>(base + kStatusOff) + i;
        d.emuRanks = (int32_t)t.nBufs;
        CollArgs &a = reinterpret_cast<CollArgs *>(base + kArgsOff)[i];
        a.in = t.in[i];
        a.out = t.out[i];
        a.count = t.count;
        a.bytes = t.bytes;
        a.elemSize = t.elemSize;
        a.op = t.op;
    }
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

    // the two-shot kernel needs (nBufs + 1) slices of ceil(bytes / nBufs), 128-byte aligned, inside one staging half
    if ((uint64_t)(nBufs + 1) * (((bytes + nBufs - 1) / nBufs + 127) & ~127ull) > kHalfBytes) {
        HCCL_ERROR("HcclLocalAllReduceNoAlloc: payload does not fit the staging half");
        return HCCL_E_INTERNAL;
    }
    CallTable t;
    memset(&t, 0, sizeof(t));
    for (uint32_t i = 0; i < nBufs; ++i) { t.in[i] = sendBufs[i]; t.out[i] = recvBufs[i]; }
    t.count = count; t.bytes = bytes; t.elemSize = DataTypeSize(dataType); t.op = (uint32_t)op; t.nBufs = nBufs;
    SmLaunch launch;
    memset(&launch, 0, sizeof(launch));
    launch.kernel = K_ALLREDUCE_TWOSHOT;
    launch.dtype = dataType;
    launch.ctas = SmCtasFor(bytes * 2 / nBufs, 4u);
    launch.args.in = sendBufs[0]; launch.args.out = recvBufs[0];
    launch.args.count = count; launch.args.bytes = bytes; launch.args.elemSize = t.elemSize; launch.args.op = t.op;
    NoAllocSetupKernel<<<1, 256, 0, stream>>>(t);
    if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    r = SmIssueEmuLaunch(reinterpret_cast<const DevComm *>(base + kCommOff), (int)nBufs, launch, reinterpret_cast<const CollArgs *>(base + kArgsOff),
                         nullptr, stream, false);
    if (r != HCCL_SUCCESS) HCCL_ERROR("HcclLocalAllReduceNoAlloc: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return r;
}

// Copies the status records of the last call (one per buffer pair: code 0 = fine, 1 = a bounded wait ran out, with the
// peer / channel / phase it was waiting for) into caller-supplied host memory, ordered after that call on `stream`.
extern "C" HcclResult HcclLocalAllReduceNoAllocStatus(void *hostRecords, uint32_t nRecords, cudaStream_t stream)
{
    if (!hostRecords) return HCCL_E_PTR;
    if (nRecords == 0 || nRecords > HCCL_NOALLOC_MAX_BUFFERS) return HCCL_E_PARA;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return HCCL_E_RUNTIME;
    char *base = nullptr;
    HcclResult r = SetupDevice(dev, &base);
    if (r != HCCL_SUCCESS) return r;
    if (cudaMemcpyAsync(hostRecords, base + kStatusOff, sizeof(DevStatus) * nRecords, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return HCCL_E_RUNTIME;
    return HCCL_SUCCESS;
}
