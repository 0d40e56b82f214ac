// Communicator-side resource API (include/hccl/hccl_res.h): state callbacks, configuration, keyed blobs, memory
// registration, the rank graph and small exchanged blobs. HCCL gets these from its communication base library
// (reference: src/common/hcomm_dlsym/hccl_host_comm_dl.h:43-58, hccl_res_dl.h:73-118, hccl_rank_graph_dl.h:38-49,
// hccl_res_expt_dl.h:25-27; the stubs its own tests use: test/stub/hccl_stub.cc:43-88); here they read the structures
// the communicator already keeps.
#include <atomic>
#include <cstring>
#include "../common/env_config.h"
#include "../common/log.h"
#include "comm.h"
#include "hccl/hccl_res.h"

using namespace hccl;

namespace {
Comm *Live(HcclComm h)
{
    Comm *c = CommFromHandle(h);
    if (!c) HCCL_ERROR("[EI0003] not a live communicator handle");
    return c;
}
std::string ExchangeKey(uint32_t rank, const char *key) { return "xchg/" + std::to_string(rank) + "/" + key; }
}  // namespace

namespace hccl {
Comm *CommFindByName(const char *name);
}

extern "C" {

HcclResult HcclCommRegCommStateCallback(HcclComm comm, HcclCommStateCallback cb, void *userData)
{
    Comm *c = Live(comm);
    if (!c || !cb) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(c->ctxMu);
    c->stateCallbacks.push_back([cb, userData](int st) { cb(userData, (HcclCommStatus)st); });
    return HCCL_SUCCESS;
}

HcclResult HcclConfigGetInfo(HcclComm comm, HcclCommConfig *config)
{
    Comm *c = Live(comm);
    if (!c || !config) return HCCL_E_PTR;
    *config = c->config;
    config->hcclBufferSize = (uint32_t)(c->devComm.cclBytes >> 20);
    config->hcclDeterministic = (uint32_t)c->env.deterministic;
    config->hcclOpExpansionMode = (uint32_t)c->env.expansionMode;
    config->hcclExecTimeoutSec = c->env.execTimeoutSec;
    config->hcclBackend = c->backend == BackendKind::CUDA ? 2 : 1;
    snprintf(config->hcclCommName, sizeof(config->hcclCommName), "%s", c->name.c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclGroupStatusGet(const char *group, HcclCommStatus *status)
{
    if (!group || !status) return HCCL_E_PTR;
    Comm *c = CommFindByName(group);
    if (!c) return HCCL_E_NOT_FOUND;
    *status = (HcclCommStatus)c->status.load();
    return HCCL_SUCCESS;
}

HcclResult HcclEngineCtxCreate(HcclComm comm, const char *tag, HcclCtxPlace place, uint64_t size, void **ptr)
{
    Comm *c = Live(comm);
    if (!c || !tag || !ptr) return HCCL_E_PTR;
    if (size == 0 || size > (1ull << 32)) return HCCL_E_PARA;
    void *have = nullptr;
    uint64_t bytes = 0;
    if (EngineCtxGet(c, tag, place == HCCL_CTX_DEVICE, &have, &bytes) == HCCL_SUCCESS) {
        HCCL_ERROR("[EI0003] engine context '%s' exists already (%llu bytes)", tag, (unsigned long long)bytes);
        return HCCL_E_PARA;
    }
    return EngineCtxCreate(c, tag, place == HCCL_CTX_DEVICE, size, ptr);
}

HcclResult HcclEngineCtxGet(HcclComm comm, const char *tag, HcclCtxPlace place, void **ptr, uint64_t *size)
{
    Comm *c = Live(comm);
    if (!c || !tag || !ptr) return HCCL_E_PTR;
    return EngineCtxGet(c, tag, place == HCCL_CTX_DEVICE, ptr, size);
}

HcclResult HcclEngineCtxCopy(HcclComm comm, const char *tag, const void *hostSrc, uint64_t size)
{
    Comm *c = Live(comm);
    if (!c || !tag || !hostSrc) return HCCL_E_PTR;
    return EngineCtxCopy(c, tag, hostSrc, size);
}

HcclResult HcclEngineCtxDestroy(HcclComm comm, const char *tag)
{
    Comm *c = Live(comm);
    if (!c || !tag) return HCCL_E_PTR;
    return EngineCtxDestroy(c, tag);
}

HcclResult HcclCommMemReg(HcclComm comm, void *addr, uint64_t size, uint64_t *windowOffset)
{
    Comm *c = Live(comm);
    if (!c || !addr || !windowOffset) return HCCL_E_PTR;
    if (size == 0) return HCCL_E_PARA;
    HcclResult r = CommRegisterWindow(c, addr, size, windowOffset);
    if (r == HCCL_E_NOT_SUPPORT)
        HCCL_ERROR("HcclCommMemReg: %p (+%llu) is outside the symmetric heap; allocate with HcclCommSymAlloc or stage through the CCL buffer",
                   addr, (unsigned long long)size);
    else if (r == HCCL_E_PARA) HCCL_ERROR("HcclCommMemReg: %p (+%llu) overlaps a window that is already registered", addr, (unsigned long long)size);
    return r;
}

HcclResult HcclCommMemDereg(HcclComm comm, void *addr)
{
    Comm *c = Live(comm);
    if (!c || !addr) return HCCL_E_PTR;
    return CommDeregisterWindow(c, addr);
}

HcclResult HcclMemAlloc(HcclComm comm, uint64_t bytes, void **ptr)
{
    Comm *c = Live(comm);
    if (!c || !ptr) return HCCL_E_PTR;
    CHK_RET(SymAlloc(c, bytes, ptr));
    uint64_t off = 0;
    HcclResult r = CommRegisterWindow(c, *ptr, bytes, &off);
    if (r != HCCL_SUCCESS) { SymFree(c, *ptr); *ptr = nullptr; }
    return r;
}

HcclResult HcclMemFree(HcclComm comm, void *ptr)
{
    Comm *c = Live(comm);
    if (!c || !ptr) return HCCL_E_PTR;
    return SymFree(c, ptr);          // windows inside the block go with it
}

// ---- allocator hooks: one attached communicator per process, looked up by handle on every call so that a hook that runs
// after the communicator's destruction (a framework's pool releasing its segments at exit) does nothing.
static std::atomic<void *> g_allocatorComm{nullptr};

}  // extern "C"
namespace hccl {
void AllocatorCommDetach(Comm *c)
{
    void *expected = c;
    g_allocatorComm.compare_exchange_strong(expected, nullptr);
}
}  // namespace hccl
extern "C" {

HcclResult HcclSetAllocatorComm(HcclComm comm)
{
    if (comm && !Live(comm)) return HCCL_E_PTR;
    g_allocatorComm.store(comm);
    return HCCL_SUCCESS;
}

HcclResult HcclGetAllocatorComm(HcclComm *comm)
{
    if (!comm) return HCCL_E_PTR;
    void *h = g_allocatorComm.load();
    *comm = CommFromHandle(h) ? h : nullptr;
    return HCCL_SUCCESS;
}

void *HcclAllocHook(long long bytes, int device, void * /*stream*/)
{
    Comm *c = CommFromHandle(g_allocatorComm.load());
    if (!c || bytes <= 0) return nullptr;
    if (c->backend == BackendKind::CUDA && device != c->device) { HCCL_ERROR("HcclAllocHook: device %d is not the communicator's device %d", device, c->device); return nullptr; }
    void *p = nullptr;
    return HcclMemAlloc(c, (uint64_t)bytes, &p) == HCCL_SUCCESS ? p : nullptr;
}

void HcclFreeHook(void *ptr, long long /*bytes*/, int /*device*/, void * /*stream*/)
{
    Comm *c = CommFromHandle(g_allocatorComm.load());
    if (c && ptr) SymFree(c, ptr);
}

HcclResult HcclRankGraphGetLayers(HcclComm comm, uint32_t *numLayers)
{
    Comm *c = Live(comm);
    if (!c || !numLayers) return HCCL_E_PTR;
    *numLayers = (uint32_t)c->topo.levels.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetRanksByLayer(HcclComm comm, uint32_t layer, uint32_t *ranks, uint32_t *num)
{
    Comm *c = Live(comm);
    if (!c || !ranks || !num) return HCCL_E_PTR;
    if (layer >= c->topo.levels.size()) return HCCL_E_PARA;
    for (const auto &group : c->topo.levels[layer]) {
        bool mine = false;
        for (uint32_t r : group) mine = mine || r == c->rank;
        if (!mine) continue;
        if (*num < group.size()) { *num = (uint32_t)group.size(); return HCCL_E_MEMORY; }
        for (size_t i = 0; i < group.size(); ++i) ranks[i] = group[i];
        *num = (uint32_t)group.size();
        return HCCL_SUCCESS;
    }
    return HCCL_E_INTERNAL;
}

HcclResult HcclRankGraphGetInstSizeListByLayer(HcclComm comm, uint32_t layer, uint32_t *sizes, uint32_t *num)
{
    Comm *c = Live(comm);
    if (!c || !sizes || !num) return HCCL_E_PTR;
    if (layer >= c->topo.levels.size()) return HCCL_E_PARA;
    const auto &groups = c->topo.levels[layer];
    if (*num < groups.size()) { *num = (uint32_t)groups.size(); return HCCL_E_MEMORY; }
    for (size_t i = 0; i < groups.size(); ++i) sizes[i] = (uint32_t)groups[i].size();
    *num = (uint32_t)groups.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetTopoTypeByLayer(HcclComm comm, uint32_t layer, HcclTopoType *type)
{
    Comm *c = Live(comm);
    if (!c || !type) return HCCL_E_PTR;
    if (layer >= c->topo.levels.size()) return HCCL_E_PARA;
    *type = layer == 0 ? (HcclTopoType)c->topo.level0Shape : HCCL_TOPO_CLOS;      // between servers: a switched network
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetLinks(HcclComm comm, uint32_t srcRank, uint32_t dstRank, HcclLinkInfo *link)
{
    Comm *c = Live(comm);
    if (!c || !link) return HCCL_E_PTR;
    if (srcRank >= c->nranks || dstRank >= c->nranks) return HCCL_E_PARA;
    memset(link, 0, sizeof(*link));
    if (srcRank == dstRank) { link->type = HCCL_LINK_NONE; return HCCL_SUCCESS; }
    for (uint32_t l = 0; l < c->topo.levels.size(); ++l) {
        for (const auto &group : c->topo.levels[l]) {
            bool a = false, b = false;
            for (uint32_t r : group) { a = a || r == srcRank; b = b || r == dstRank; }
            if (!(a && b)) continue;
            link->layer = l;
            if (l == 0) {
                link->type = c->backend == BackendKind::CUDA ? (HcclLinkType)c->topo.level0Link : HCCL_LINK_SHM;
                link->peerAccess = c->topo.allPeersDirect ? 1u : 0u;
            } else {
                link->type = HCCL_LINK_NET;
                link->peerAccess = c->backend == BackendKind::CUDA ? 0u : 1u;    // simulated servers share host memory
            }
            link->bandwidthGBs = l < c->topo.levelBandwidth.size() ? c->topo.levelBandwidth[l] : 0.0;
            return HCCL_SUCCESS;
        }
    }
    // no common group at any layer: reachable only through two hops (e.g. different local index on different servers)
    link->type = HCCL_LINK_NET;
    link->layer = (uint32_t)c->topo.levels.size();
    return HCCL_SUCCESS;
}

HcclResult HcclCommAddExchangeInfo(HcclComm comm, const char *key, const void *data, uint32_t size)
{
    Comm *c = Live(comm);
    if (!c || !key || (!data && size)) return HCCL_E_PTR;
    if (size > 4096) { HCCL_ERROR("[EI0003] exchange info is limited to 4096 bytes (got %u)", size); return HCCL_E_PARA; }
    return c->boot->Put(ExchangeKey(c->rank, key), data, size);
}

HcclResult HcclCommGetExchangeInfo(HcclComm comm, uint32_t rank, const char *key, void *data, uint32_t *size)
{
    Comm *c = Live(comm);
    if (!c || !key || !data || !size) return HCCL_E_PTR;
    if (rank >= c->nranks) return HCCL_E_PARA;
    std::vector<uint8_t> v;
    CHK_RET(c->boot->Get(ExchangeKey(rank, key), &v, c->env.connectTimeoutSec));
    if (v.size() > *size) { *size = (uint32_t)v.size(); return HCCL_E_MEMORY; }
    if (!v.empty()) memcpy(data, v.data(), v.size());
    *size = (uint32_t)v.size();
    return HCCL_SUCCESS;
}

}  // extern "C"
