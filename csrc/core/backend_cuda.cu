// CUDA backend of the communicator: symmetric heap from VMM allocations shared as POSIX file descriptors,
// optional NVSwitch multicast (NVLS) mapping over the same memory, pinned status word, device copy of DevComm.
//
// Driver entry points are fetched through cudaGetDriverEntryPoint so the library has no link-time dependency on
// libcuda and still loads on machines without a driver (where only the host simulation backend is usable).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstring>
#include <unistd.h>
#include "../common/log.h"
#include "comm.h"

namespace hccl {

void HeapLayoutForBackend(Comm *c, uint64_t granularity);

namespace {

struct DriverApi {
    bool ok = false;
    CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
    CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
    CUresult (*DeviceGet)(CUdevice *, int);
    CUresult (*GetErrorString)(CUresult, const char **);
};

DriverApi &Drv()
{
    static DriverApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        bool ok = true;
        auto get = [&](const char *name, void **fn) {
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || *fn == nullptr) {
                ok = false;
                (void)cudaGetLastError();
            }
        };
        get("cuMemGetAllocationGranularity", (void **)&api.MemGetAllocationGranularity);
        get("cuMemCreate", (void **)&api.MemCreate);
        get("cuMemRelease", (void **)&api.MemRelease);
        get("cuMemExportToShareableHandle", (void **)&api.MemExportToShareableHandle);
        get("cuMemImportFromShareableHandle", (void **)&api.MemImportFromShareableHandle);
        get("cuMemAddressReserve", (void **)&api.MemAddressReserve);
        get("cuMemAddressFree", (void **)&api.MemAddressFree);
        get("cuMemMap", (void **)&api.MemMap);
        get("cuMemUnmap", (void **)&api.MemUnmap);
        get("cuMemSetAccess", (void **)&api.MemSetAccess);
        get("cuMulticastCreate", (void **)&api.MulticastCreate);
        get("cuMulticastAddDevice", (void **)&api.MulticastAddDevice);
        get("cuMulticastBindMem", (void **)&api.MulticastBindMem);
        get("cuMulticastUnbind", (void **)&api.MulticastUnbind);
        get("cuMulticastGetGranularity", (void **)&api.MulticastGetGranularity);
        get("cuDeviceGetAttribute", (void **)&api.DeviceGetAttribute);
        get("cuDeviceGet", (void **)&api.DeviceGet);
        get("cuGetErrorString", (void **)&api.GetErrorString);
        api.ok = ok;
    });
    return api;
}

const char *CuErr(CUresult r)
{
    const char *s = nullptr;
    if (Drv().GetErrorString) Drv().GetErrorString(r, &s);
    return s ? s : "unknown";
}

#define CU_CHK(call)                                                                       \
    do {                                                                                   \
        CUresult _r = (call);                                                              \
        if (_r != CUDA_SUCCESS) {                                                          \
            HCCL_ERROR("driver call %s failed: %d (%s)", #call, (int)_r, CuErr(_r));       \
            return HCCL_E_DRV;                                                             \
        }                                                                                  \
    } while (0)
#define RT_CHK(call)                                                                       \
    do {                                                                                   \
        cudaError_t _e = (call);                                                           \
        if (_e != cudaSuccess) {                                                           \
            HCCL_ERROR("runtime call %s failed: %s", #call, cudaGetErrorString(_e));       \
            return HCCL_E_RUNTIME;                                                         \
        }                                                                                  \
    } while (0)

struct CudaHeapState {
    CUmemGenericAllocationHandle local = 0;
    std::vector<CUmemGenericAllocationHandle> peers;
    std::vector<CUdeviceptr> vas;
    CUmemGenericAllocationHandle mc = 0;
    CUdeviceptr mcVa = 0;
    bool mcBound = false, mcAdded = false;
    CUdevice cuDev = 0;
    uint64_t bytes = 0;
    int localFd = -1;
    cudaStream_t dfxStream = nullptr;   // private stream of the diagnostic copies
};

}  // namespace

bool CudaDeviceAvailable(int *currentDevice)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); return false; }
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    if (currentDevice) *currentDevice = d;
    return true;
}

void CudaFillRankDesc(int dev, RankDesc *d)
{
    cudaDeviceGetPCIBusId(d->busId, sizeof(d->busId), dev);
    d->nvlsCapable = 0;
    DriverApi &api = Drv();
    if (api.ok) {
        CUdevice cd;
        int v = 0;
        if (api.DeviceGet(&cd, dev) == CUDA_SUCCESS && api.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) == CUDA_SUCCESS) d->nvlsCapable = (uint32_t)v;
    }
}

// This rank's view of its links: peer access and its quality from the CUDA runtime, NVLink or not from NVML.
void CudaFillLinkRow(int dev, const std::vector<RankDesc> &all, uint32_t myRank, LinkRow *row)
{
    memset(row, 0, sizeof(*row));
    (void)NvmlProbePair(all[myRank].busId, nullptr, nullptr, &row->nvlinkActive, &row->nvlinkVersion);
    for (uint32_t r = 0; r < all.size() && r < (uint32_t)kTopoMaxRanks; ++r) {
        row->perfRank[r] = 255;
        if (r == myRank) { row->type[r] = (uint8_t)LinkType::SHM; continue; }
        if (all[r].hostHash != all[myRank].hostHash || all[r].deviceId < 0) { row->type[r] = (uint8_t)LinkType::NET; continue; }
        if (all[r].deviceId == dev) { row->type[r] = (uint8_t)LinkType::SHM; row->perfRank[r] = 0; row->atomics[r] = 1; continue; }
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, dev, all[r].deviceId) != cudaSuccess) { (void)cudaGetLastError(); can = 0; }
        if (!can) { row->type[r] = (uint8_t)LinkType::NONE; continue; }
        int perf = 255, atom = 0;
        if (cudaDeviceGetP2PAttribute(&perf, cudaDevP2PAttrPerformanceRank, dev, all[r].deviceId) != cudaSuccess) { (void)cudaGetLastError(); perf = 255; }
        if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, dev, all[r].deviceId) != cudaSuccess) { (void)cudaGetLastError(); atom = 0; }
        row->perfRank[r] = (uint8_t)std::min(perf, 255);
        row->atomics[r] = (uint8_t)(atom != 0);
        int nvl = -1;
        (void)NvmlProbePair(all[myRank].busId, all[r].busId, &nvl, nullptr, nullptr);
        // NVML decides when it can; otherwise native atomics over the link mean NVLink (PCIe peers have none)
        row->type[r] = (uint8_t)((nvl == 1 || (nvl < 0 && atom)) ? LinkType::NVLINK : LinkType::PCIE);
    }
}

HcclResult CudaAllocDevice(void **p, uint64_t bytes) { RT_CHK(cudaMalloc(p, bytes)); return HCCL_SUCCESS; }
void CudaFreeDevice(void *p) { if (p) cudaFree(p); }
HcclResult CudaCopyToDevice(void *dst, const void *src, uint64_t bytes) { RT_CHK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice)); return HCCL_SUCCESS; }

static HcclResult MapHandle(DriverApi &api, CUmemGenericAllocationHandle h, uint64_t bytes, uint64_t gran, CUdevice dev, CUdeviceptr *va)
{
    CU_CHK(api.MemAddressReserve(va, bytes, gran, 0, 0));
    CU_CHK(api.MemMap(*va, bytes, 0, h, 0));
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CU_CHK(api.MemSetAccess(*va, bytes, &acc, 1));
    return HCCL_SUCCESS;
}

static HcclResult SetupMulticast(Comm *c, CudaHeapState *st, DriverApi &api, uint64_t gran)
{
    CUmulticastObjectProp mp{};
    mp.numDevices = c->nranks;
    mp.size = c->heapBytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    int rootFd = -1;
    int32_t okLocal = 1;
    if (c->rank == 0) {
        CUresult r = api.MulticastCreate(&st->mc, &mp);
        if (r == CUDA_SUCCESS) r = api.MemExportToShareableHandle(&rootFd, st->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        if (r != CUDA_SUCCESS) { HCCL_WARNING("NVLS: multicast object creation failed (%s); using peer loads/stores", CuErr(r)); okLocal = 0; }
    }
    std::vector<int32_t> oks(c->nranks);
    CHK_RET(c->boot->AllGather(&okLocal, 4, oks.data()));
    if (!oks[0]) { if (st->mc) { api.MemRelease(st->mc); st->mc = 0; } return HCCL_E_UNAVAIL; }
    std::vector<std::vector<int>> fds;
    std::vector<int> mine;
    if (c->rank == 0) mine.push_back(rootFd);
    CHK_RET(FdExchange::AllGatherFds(c->boot->Nonce(), "mc" + std::to_string(c->commId & 0xffff), c->rank, c->nranks, mine, &fds,
                                     c->boot.get(), c->env.connectTimeoutSec));
    if (c->rank != 0) {
        if (fds[0].size() != 1) okLocal = 0;
        else {
            CUresult r = api.MemImportFromShareableHandle(&st->mc, (void *)(uintptr_t)fds[0][0], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            close(fds[0][0]);
            if (r != CUDA_SUCCESS) { HCCL_WARNING("NVLS: import failed (%s)", CuErr(r)); okLocal = 0; st->mc = 0; }
        }
    } else if (rootFd >= 0) close(rootFd);
    if (okLocal) {
        CUresult r = api.MulticastAddDevice(st->mc, st->cuDev);
        if (r != CUDA_SUCCESS) { HCCL_WARNING("NVLS: add device failed (%s)", CuErr(r)); okLocal = 0; }
        else st->mcAdded = true;
    }
    CHK_RET(c->boot->AllGather(&okLocal, 4, oks.data()));   // all devices added before anyone binds
    bool all = true;
    for (int32_t v : oks) all = all && v;
    if (all) {
        CUresult r = api.MulticastBindMem(st->mc, 0, st->local, 0, c->heapBytes, 0);
        if (r != CUDA_SUCCESS) { HCCL_WARNING("NVLS: bind failed (%s)", CuErr(r)); okLocal = 0; }
        else st->mcBound = true;
        if (okLocal) {
            if (MapHandle(api, st->mc, c->heapBytes, gran, st->cuDev, &st->mcVa) != HCCL_SUCCESS) { okLocal = 0; st->mcVa = 0; }
        }
    }
    CHK_RET(c->boot->AllGather(&okLocal, 4, oks.data()));
    all = true;
    for (int32_t v : oks) all = all && v;
    if (!all) {
        if (st->mcVa) { api.MemUnmap(st->mcVa, c->heapBytes); api.MemAddressFree(st->mcVa, c->heapBytes); st->mcVa = 0; }
        if (st->mcBound) { api.MulticastUnbind(st->mc, st->cuDev, 0, c->heapBytes); st->mcBound = false; }
        if (st->mc) { api.MemRelease(st->mc); st->mc = 0; }
        return HCCL_E_UNAVAIL;
    }
    c->mcHeap = (char *)st->mcVa;
    return HCCL_SUCCESS;
}

HcclResult CudaBackendInit(Comm *c)
{
    DriverApi &api = Drv();
    RT_CHK(cudaSetDevice(c->device));
    RT_CHK(cudaFree(nullptr));
    if (!api.ok) { HCCL_ERROR("CUDA driver entry points for virtual memory management are unavailable"); return HCCL_E_UNAVAIL; }
    auto *st = new CudaHeapState();
    c->backendState = st;
    CU_CHK(api.DeviceGet(&st->cuDev, c->device));

    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = c->device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    CU_CHK(api.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    bool wantNvls = c->env.nvlsEnable && c->nranks > 1 && c->topo.nvlsSupported;
    if (wantNvls) {
        CUmulticastObjectProp mp{};
        mp.numDevices = c->nranks;
        mp.size = 1ull << 30;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg = 0;
        if (api.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    HeapLayoutForBackend(c, gran);
    st->bytes = c->heapBytes;

    CU_CHK(api.MemCreate(&st->local, c->heapBytes, &prop, 0));
    CU_CHK(api.MemExportToShareableHandle(&st->localFd, st->local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    std::vector<std::vector<int>> fds;
    CHK_RET(FdExchange::AllGatherFds(c->boot->Nonce(), "heap" + std::to_string(c->commId & 0xffff), c->rank, c->nranks, {st->localFd},
                                     &fds, c->boot.get(), c->env.connectTimeoutSec));
    st->peers.assign(c->nranks, 0);
    st->vas.assign(c->nranks, 0);
    c->heap.assign(c->nranks, nullptr);
    for (uint32_t r = 0; r < c->nranks; ++r) {
        if (r == c->rank) st->peers[r] = st->local;
        else {
            if (fds[r].size() != 1) return HCCL_E_INTERNAL;
            CUresult rc = api.MemImportFromShareableHandle(&st->peers[r], (void *)(uintptr_t)fds[r][0], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            close(fds[r][0]);
            if (rc != CUDA_SUCCESS) { HCCL_ERROR("import of rank %u's heap failed: %s", r, CuErr(rc)); return HCCL_E_DRV; }
        }
        HcclResult mr = MapHandle(api, st->peers[r], c->heapBytes, gran, st->cuDev, &st->vas[r]);
        if (mr != HCCL_SUCCESS) { HCCL_ERROR("mapping rank %u's heap failed (no peer access between the devices?)", r); return HCCL_E_UNAVAIL; }
        c->heap[r] = (char *)st->vas[r];
        c->devComm.heap[r] = c->heap[r];
    }
    close(st->localFd);
    st->localFd = -1;
    RT_CHK(cudaMemset(c->heap[c->rank], 0, kHeapHeaderBytes));
    RT_CHK(cudaDeviceSynchronize());

    if (wantNvls) {
        LogPushErrorToWarn();
        HcclResult nr = SetupMulticast(c, st, api, gran);
        LogPopErrorToWarn();
        if (nr != HCCL_SUCCESS && nr != HCCL_E_UNAVAIL) return nr;
    }
    c->devComm.mcHeap = c->mcHeap;

    RT_CHK(cudaHostAlloc((void **)&c->hostStatus, sizeof(DevStatus), cudaHostAllocMapped | cudaHostAllocPortable));
    memset(c->hostStatus, 0, sizeof(DevStatus));
    DevStatus *devStatus = nullptr;
    RT_CHK(cudaHostGetDevicePointer((void **)&devStatus, c->hostStatus, 0));
    c->devComm.status = devStatus;
    RT_CHK(cudaHostAlloc((void **)&c->hostProgress, 64, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(c->hostProgress, 0, 64);
    RT_CHK(cudaHostGetDevicePointer((void **)&c->devComm.progress, c->hostProgress, 0));
    {
        const char *e = getenv("HCCL_DEVICE_TRACE");
        c->devComm.traceOn = e ? atoi(e) != 0 : 1;
    }
    RT_CHK(cudaMalloc((void **)&c->devCommPtr, sizeof(DevComm)));
    RT_CHK(cudaMemcpy(c->devCommPtr, &c->devComm, sizeof(DevComm), cudaMemcpyHostToDevice));
    return c->boot->Barrier();
}

// Waits for every kernel and copy this rank has queued on its device. Called before the host barriers of destroy and
// resume: once all ranks have passed such a barrier no kernel anywhere can still touch a peer's heap or flags.
HcclResult CudaBackendQuiesce(Comm *c)
{
    RT_CHK(cudaSetDevice(c->device));
    RT_CHK(cudaDeviceSynchronize());
    return HCCL_SUCCESS;
}

HcclResult CudaBackendResetFlags(Comm *c)
{
    RT_CHK(cudaSetDevice(c->device));
    RT_CHK(cudaDeviceSynchronize());
    RT_CHK(cudaMemset(c->heap[c->rank], 0, kHeapHeaderBytes));
    RT_CHK(cudaDeviceSynchronize());
    if (c->hostProgress) *c->hostProgress = 0;
    c->devOpIssued = 0;
    return HCCL_SUCCESS;
}

// Copies the first `bytes` of this rank's heap (control block, trace ring, flag arena) to host memory on a private
// stream, so that it neither waits for nor delays the caller's streams.
HcclResult CudaReadHeapHeader(Comm *c, void *hostDst, uint64_t bytes)
{
    auto *st = (CudaHeapState *)c->backendState;
    if (st == nullptr || bytes > kHeapHeaderBytes) return HCCL_E_PARA;
    RT_CHK(cudaSetDevice(c->device));
    if (!st->dfxStream) RT_CHK(cudaStreamCreateWithFlags(&st->dfxStream, cudaStreamNonBlocking));
    RT_CHK(cudaMemcpyAsync(hostDst, c->heap[c->rank], bytes, cudaMemcpyDeviceToHost, st->dfxStream));
    RT_CHK(cudaStreamSynchronize(st->dfxStream));
    return HCCL_SUCCESS;
}

void CudaBackendDestroy(Comm *c)
{
    auto *st = (CudaHeapState *)c->backendState;
    if (st == nullptr) return;
    DriverApi &api = Drv();
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    // Multicast first: unmap the multicast VA, unbind this device's memory, drop the object. CommDestroy has drained
    // every rank's device BEFORE its host barrier, so no peer kernel can still read or reduce through this binding.
    if (st->mcVa) { api.MemUnmap(st->mcVa, st->bytes); api.MemAddressFree(st->mcVa, st->bytes); }
    if (st->mcBound) api.MulticastUnbind(st->mc, st->cuDev, 0, st->bytes);
    if (st->mc) api.MemRelease(st->mc);
    for (size_t r = 0; r < st->vas.size(); ++r) {
        if (st->vas[r]) { api.MemUnmap(st->vas[r], st->bytes); api.MemAddressFree(st->vas[r], st->bytes); }
        if (st->peers[r] && r != c->rank) api.MemRelease(st->peers[r]);
    }
    if (st->local) api.MemRelease(st->local);
    if (st->localFd >= 0) close(st->localFd);
    if (c->devCommPtr) cudaFree(c->devCommPtr);
    if (c->hostStatus) cudaFreeHost(c->hostStatus);
    if (c->hostProgress) cudaFreeHost(c->hostProgress);
    c->hostProgress = nullptr;
    if (st->dfxStream) cudaStreamDestroy(st->dfxStream);
    c->devCommPtr = nullptr;
    c->hostStatus = nullptr;
    c->mcHeap = nullptr;
    delete st;
    c->backendState = nullptr;
}

}  // namespace hccl
