// Read-only NVLink discovery through NVML, loaded at run time (no link-time dependency; nothing is ever set).
//
// The CUDA runtime tells whether two devices can access each other and how good the path is; NVML adds whether that path is
// NVLink (nvmlDeviceGetP2PStatus, NVLINK capability) and how many of a device's links are up. Both feed LinkRow, the per-rank
// link description the topology builder counts (reference: pair-link counting in src/ops/op_common/topo/topo_host.cc:280-332).
// HCCL_NVML_LIB names the library to load (default libnvidia-ml.so.1); tests point it at a stand-in that describes a box
// with a missing link.
#include <dlfcn.h>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "../common/log.h"
#include "topo_info.h"

namespace hccl {

namespace {
using NvmlDevice = void *;
struct NvmlApi {
    void *lib = nullptr;
    int (*init)() = nullptr;
    int (*handleByBusId)(const char *, NvmlDevice *) = nullptr;
    int (*p2pStatus)(NvmlDevice, NvmlDevice, int, int *) = nullptr;
    int (*nvlinkState)(NvmlDevice, unsigned, int *) = nullptr;
    int (*nvlinkVersion)(NvmlDevice, unsigned, unsigned *) = nullptr;
    bool ok = false;
};
std::mutex g_mu;
NvmlApi g_api;
std::string g_loadedFrom;

NvmlApi &Nvml()
{
    std::lock_guard<std::mutex> lk(g_mu);
    const char *path = getenv("HCCL_NVML_LIB");
    std::string want = path && *path ? path : "libnvidia-ml.so.1";
    if (g_api.lib && want == g_loadedFrom) return g_api;
    g_api = NvmlApi();
    g_loadedFrom = want;
    g_api.lib = dlopen(want.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!g_api.lib) return g_api;
    g_api.init = (int (*)())dlsym(g_api.lib, "nvmlInit_v2");
    g_api.handleByBusId = (int (*)(const char *, NvmlDevice *))dlsym(g_api.lib, "nvmlDeviceGetHandleByPciBusId_v2");
    g_api.p2pStatus = (int (*)(NvmlDevice, NvmlDevice, int, int *))dlsym(g_api.lib, "nvmlDeviceGetP2PStatus");
    g_api.nvlinkState = (int (*)(NvmlDevice, unsigned, int *))dlsym(g_api.lib, "nvmlDeviceGetNvLinkState");
    g_api.nvlinkVersion = (int (*)(NvmlDevice, unsigned, unsigned *))dlsym(g_api.lib, "nvmlDeviceGetNvLinkVersion");
    g_api.ok = g_api.init && g_api.handleByBusId && g_api.init() == 0;
    return g_api;
}
}  // namespace

// nvlinkP2P: 1 = NVLink peer-to-peer between the two devices, 0 = not, -1 = NVML cannot tell. activeLinks / version describe
// device A (0 = unknown).
HcclResult NvmlProbePair(const char *busIdA, const char *busIdB, int *nvlinkP2P, uint32_t *activeLinks, uint32_t *version)
{
    if (nvlinkP2P) *nvlinkP2P = -1;
    if (activeLinks) *activeLinks = 0;
    if (version) *version = 0;
    NvmlApi &n = Nvml();
    if (!n.ok) return HCCL_E_UNAVAIL;
    NvmlDevice a = nullptr, b = nullptr;
    if (n.handleByBusId(busIdA, &a) != 0) return HCCL_E_NOT_FOUND;
    if (busIdB && *busIdB && n.p2pStatus && n.handleByBusId(busIdB, &b) == 0 && nvlinkP2P) {
        int status = -1;
        constexpr int kCapNvlink = 2;      // NVML_P2P_CAPS_INDEX_NVLINK
        if (n.p2pStatus(a, b, kCapNvlink, &status) == 0) *nvlinkP2P = status == 0 ? 1 : 0;   // NVML_P2P_STATUS_OK == 0
    }
    if (n.nvlinkState && activeLinks) {
        for (unsigned l = 0; l < 18; ++l) {
            int up = 0;
            if (n.nvlinkState(a, l, &up) != 0) break;
            if (up) ++*activeLinks;
        }
    }
    if (n.nvlinkVersion && version) (void)n.nvlinkVersion(a, 0, version);
    return HCCL_SUCCESS;
}

}  // namespace hccl
