// extern "C" communicator management (see include/hccl/hccl_comm.h).
#include <cstring>
#include <fstream>
#include <sstream>
#include <thread>
#include "../common/dtype.h"
#include "../common/json.h"
#include "../common/log.h"
#include "../exec/executor.h"
#include "comm.h"
#include "../exec/op_common.h"
#include "hccl/hccl_comm.h"

using namespace hccl;

namespace hccl {
namespace mc2 { void DropWorkspace(Comm *c); }
extern HcclResult CudaSetDeviceChecked(int dev);
HcclResult BootstrapFixedRootInfo(const std::string &ip, uint32_t port, uint64_t nonce, bool listen, HcclRootInfo *out);
}

extern "C" {

void HcclCommConfigInit(HcclCommConfig *config)
{
    if (!config) return;
    memset(config, 0, sizeof(*config));
    config->size = sizeof(HcclCommConfig);
    config->magic = HCCL_COMM_CONFIG_MAGIC;
    config->version = 1;
    config->hcclBufferSize = 0;
    config->hcclDeterministic = HCCL_CONFIG_NOT_SET;
    config->hcclOpExpansionMode = 0;
    config->hcclExecTimeoutSec = 0;
    config->hcclBackend = 0;
}

HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo)
{
    if (!rootInfo) return HCCL_E_PTR;
    return Bootstrap::CreateRootInfo(rootInfo);
}

HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, const HcclCommConfig *config, HcclComm *comm)
{
    if (!comm) return HCCL_E_PTR;
    Comm *c = nullptr;
    HcclResult r;
    try { r = CommCreate(nRanks, rootInfo, rank, config, &c); }
    catch (const std::exception &e) { HCCL_ERROR("HcclCommInitRootInfo: %s", e.what()); return HCCL_E_INTERNAL; }
    if (r != HCCL_SUCCESS) return r;
    *comm = c;
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm)
{
    return HcclCommInitRootInfoConfig(nRanks, rootInfo, rank, nullptr, comm);
}

// Rank table (HCCL "ranktable" JSON, reference schema: docs/zh/user_guide/cluster_info_config/rank_table_config_a2.md:10-52):
//   {"status":"completed","version":"1.0","server_count":"1",
//    "server_list":[{"server_id":"<host ip>","device":[{"device_id":"0","rank_id":"0"}, ...]}]}
// The first server's id is the bootstrap address; the port is HCCL_IF_BASE_PORT (default 60000) and the rendezvous
// nonce is a hash of the file, so every rank derives the same root info without out-of-band exchange.
HcclResult HcclCommInitClusterInfoConfig(const char *clusterInfo, uint32_t rank, const HcclCommConfig *config, HcclComm *comm)
{
    if (!clusterInfo || !comm) return HCCL_E_PTR;
    InitEnvConfig();
    std::ifstream f(clusterInfo);
    if (!f) { HCCL_ERROR("rank table %s cannot be opened", clusterInfo); return HCCL_E_OPEN_FILE_FAILURE; }
    std::stringstream ss;
    ss << f.rdbuf();
    std::string text = ss.str();
    uint32_t nranks = 0;
    std::string rootIp;
    int myDevice = -1;
    int myServer = -1;                       // position of this rank's server in server_list
    std::string myServerId;
    int mySuperPod = 0;
    try {
        JsonValue root = JsonParser(text).Parse();
        const JsonValue *status = root.Get("status");
        if (status && status->str != "completed") { HCCL_ERROR("rank table status is '%s', expected 'completed'", status->str.c_str()); return HCCL_E_PARA; }
        const JsonValue *servers = root.Get("server_list");
        if (!servers || servers->kind != JsonValue::ARR || servers->arr.empty()) { HCCL_ERROR("rank table has no server_list"); return HCCL_E_PARA; }
        const JsonValue *sc = root.Get("server_count");
        long long scv;
        if (sc && sc->AsInt(&scv) && (size_t)scv != servers->arr.size()) { HCCL_ERROR("rank table: server_count %lld but %zu servers listed", scv, servers->arr.size()); return HCCL_E_PARA; }
        std::vector<bool> seen;
        int serverOrdinal = -1;
        for (const JsonValue &s : servers->arr) {
            ++serverOrdinal;
            const JsonValue *sid = s.Get("server_id");
            if (rootIp.empty() && sid) rootIp = sid->str;
            const JsonValue *devs = s.Get("device");
            if (!devs || devs->kind != JsonValue::ARR) { HCCL_ERROR("rank table: server without device list"); return HCCL_E_PARA; }
            for (const JsonValue &d : devs->arr) {
                long long rid, did = -1;
                const JsonValue *r = d.Get("rank_id");
                if (!r || !r->AsInt(&rid) || rid < 0) { HCCL_ERROR("rank table: device without rank_id"); return HCCL_E_PARA; }
                if (const JsonValue *dv = d.Get("device_id")) dv->AsInt(&did);
                if ((size_t)rid >= seen.size()) seen.resize(rid + 1, false);
                if (seen[rid]) { HCCL_ERROR("rank table: rank_id %lld listed twice", rid); return HCCL_E_PARA; }
                seen[rid] = true;
                if ((uint32_t)rid == rank) { myDevice = (int)did; myServer = serverOrdinal; if (sid) myServerId = sid->str; }
                ++nranks;
            }
        }
        for (size_t i = 0; i < seen.size(); ++i) if (!seen[i]) { HCCL_ERROR("rank table: rank_id %zu missing", i); return HCCL_E_PARA; }
        // optional "super_pod_list": [{"super_pod_id": "0", "server_list": [{"server_id": "..."}]}] (the reference's tables for machines
        // with super-pods, docs/zh/user_guide/cluster_info_config/rank_table_config_a3.md)
        if (const JsonValue *pods = root.Get("super_pod_list"))
            if (pods->kind == JsonValue::ARR) {
                int podOrdinal = -1;
                for (const JsonValue &pod : pods->arr) {
                    ++podOrdinal;
                    const JsonValue *sl = pod.Get("server_list");
                    if (!sl || sl->kind != JsonValue::ARR) continue;
                    for (const JsonValue &sv : sl->arr) {
                        const JsonValue *sid = sv.Get("server_id");
                        if (sid && !myServerId.empty() && sid->str == myServerId) mySuperPod = podOrdinal;
                    }
                }
            }
    } catch (const std::exception &e) {
        HCCL_ERROR("rank table %s: %s", clusterInfo, e.what());
        return HCCL_E_PARA;
    }
    if (rank >= nranks) { HCCL_ERROR("[EI0003] rank %u is not in the rank table (%u ranks)", rank, nranks); return HCCL_E_PARA; }
    uint64_t nonce = 1469598103934665603ull;
    for (char ch : text) nonce = (nonce ^ (uint8_t)ch) * 1099511628211ull;
    uint32_t port = GetEnvConfig().ifBasePort ? GetEnvConfig().ifBasePort : 60000;
    if (rootIp.empty() || rootIp.find_first_not_of("0123456789.") != std::string::npos) rootIp = GetEnvConfig().ifIp;
    HcclRootInfo info;
    CHK_RET(BootstrapFixedRootInfo(rootIp, port, nonce, rank == 0, &info));
    int dev;
    if (myDevice >= 0 && CudaDeviceAvailable(&dev) && !(config && config->hcclBackend == 1)) CHK_RET(CudaSetDeviceChecked(myDevice));
    // The host simulation has no hosts to tell servers apart by: there the table's server list places the ranks (GPUs sit where their
    // host says, and the table is expected to say the same).
    RankDesc placed{};
    placed.serverId = (uint32_t)std::max(myServer, 0);
    placed.superPodId = (uint32_t)mySuperPod;
    placed.hostHash = 0x9e3779b97f4a7c15ull * (placed.serverId + 1);
    SetInheritedPlacement(&placed, true);
    HcclResult r = HcclCommInitRootInfoConfig(nranks, &info, rank, config, comm);
    SetInheritedPlacement(nullptr);
    return r;
}

HcclResult HcclCommInitClusterInfo(const char *clusterInfo, uint32_t rank, HcclComm *comm)
{
    return HcclCommInitClusterInfoConfig(clusterInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitAll(uint32_t ndev, int32_t *devices, HcclComm *comms)
{
    if (!comms) return HCCL_E_PTR;
    if (ndev == 0) return HCCL_E_PARA;
    InitEnvConfig();
    HcclRootInfo info;
    CHK_RET(HcclGetRootInfo(&info));
    int cur;
    bool cuda = CudaDeviceAvailable(&cur);
    if (const char *e = getenv("HCCL_BACKEND")) if (!strcasecmp(e, "sim") || !strcasecmp(e, "host")) cuda = false;
    if (cuda && devices) {
        for (uint32_t i = 0; i < ndev; ++i)
            for (uint32_t j = i + 1; j < ndev; ++j)
                if (devices[i] == devices[j]) { HCCL_ERROR("[EI0003] HcclCommInitAll: device %d listed twice", devices[i]); return HCCL_E_PARA; }
    }
    std::vector<HcclResult> res(ndev, HCCL_SUCCESS);
    std::vector<std::thread> th;
    for (uint32_t r = 0; r < ndev; ++r)
        th.emplace_back([&, r] {
            if (cuda) { HcclResult s = CudaSetDeviceChecked(devices ? devices[r] : (int)r); if (s != HCCL_SUCCESS) { res[r] = s; return; } }
            res[r] = HcclCommInitRootInfo(ndev, &info, r, &comms[r]);
        });
    for (auto &t : th) t.join();
    for (HcclResult r : res) if (r != HCCL_SUCCESS) return r;
    return HCCL_SUCCESS;
}

HcclResult HcclCreateSubCommConfig(HcclComm *comm, uint32_t rankNum, uint32_t *rankIds, uint64_t subCommId, uint32_t subCommRankId,
                                   HcclCommConfig *config, HcclComm *subComm)
{
    if (!comm || !subComm) return HCCL_E_PTR;
    Comm *parent = CommFromHandle(*comm);
    if (!parent) return HCCL_E_PARA;
    if (rankIds == nullptr || rankNum == 0) { *subComm = nullptr; return HCCL_SUCCESS; }   // this rank is not a member
    if (subCommRankId >= rankNum || rankIds[subCommRankId] != parent->rank) { HCCL_ERROR("[EI0003] sub comm: rankIds[%u] must be this rank (%u)", subCommRankId, parent->rank); return HCCL_E_PARA; }
    for (uint32_t i = 0; i < rankNum; ++i) if (rankIds[i] >= parent->nranks) return HCCL_E_PARA;
    std::string key = "subcomm-" + std::to_string(subCommId);
    HcclRootInfo info;
    if (subCommRankId == 0) {
        CHK_RET(HcclGetRootInfo(&info));
        CHK_RET(parent->boot->Put(key, &info, sizeof(info)));
    } else {
        std::vector<uint8_t> v;
        CHK_RET(parent->boot->Get(key, &v, parent->env.connectTimeoutSec));
        if (v.size() != sizeof(info)) return HCCL_E_INTERNAL;
        memcpy(&info, v.data(), sizeof(info));
    }
    const bool known = parent->rank < parent->topo.ranks.size();
    if (known) SetInheritedPlacement(&parent->topo.ranks[parent->rank]);
    HcclResult r = HcclCommInitRootInfoConfig(rankNum, &info, subCommRankId, config, subComm);
    SetInheritedPlacement(nullptr);
    return r;
}

HcclResult HcclCommDestroy(HcclComm comm)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return comm ? HCCL_E_PARA : HCCL_E_PTR;
    PlanCache::Drop(c);
    mc2::DropWorkspace(c);
    return CommDestroy(c);
}

HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !rankSize) return HCCL_E_PTR;
    *rankSize = c->nranks;
    return HCCL_SUCCESS;
}
HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !rank) return HCCL_E_PTR;
    *rank = c->rank;
    return HCCL_SUCCESS;
}
HcclResult HcclGetCommName(HcclComm comm, char *commName)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !commName) return HCCL_E_PTR;
    snprintf(commName, HCCL_COMM_NAME_MAX, "%s", c->name.c_str());
    return HCCL_SUCCESS;
}
HcclResult HcclGetHcclBuffer(HcclComm comm, void **addr, uint64_t *size)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !addr || !size) return HCCL_E_PTR;
    *addr = c->heap[c->rank] + c->devComm.cclOff[0];
    *size = c->devComm.cclBytes;
    return HCCL_SUCCESS;
}

const char *HcclGetErrorString(HcclResult code)
{
    switch (code) {
        case HCCL_SUCCESS: return "success";
        case HCCL_E_PARA: return "invalid parameter";
        case HCCL_E_PTR: return "null pointer";
        case HCCL_E_MEMORY: return "memory error";
        case HCCL_E_INTERNAL: return "internal error";
        case HCCL_E_NOT_SUPPORT: return "not supported";
        case HCCL_E_NOT_FOUND: return "not found";
        case HCCL_E_UNAVAIL: return "resource unavailable";
        case HCCL_E_SYSCALL: return "system call failed";
        case HCCL_E_TIMEOUT: return "timeout";
        case HCCL_E_OPEN_FILE_FAILURE: return "cannot open file";
        case HCCL_E_TCP_CONNECT: return "tcp connect failed";
        case HCCL_E_TCP_TRANSFER: return "tcp transfer failed";
        case HCCL_E_RUNTIME: return "CUDA runtime error";
        case HCCL_E_DRV: return "CUDA driver error";
        case HCCL_E_REMOTE: return "a remote rank failed";
        case HCCL_E_SUSPENDING: return "communicator suspended";
        case HCCL_E_OOM: return "out of memory";
        default: return "error";
    }
}

HcclResult HcclCommGetStatus(HcclComm comm, HcclCommStatus *status)
{
    Comm *c = CommFromHandle(comm);
    if (!status) return HCCL_E_PTR;
    if (!c) { *status = HCCL_COMM_STATUS_INVALID; return HCCL_SUCCESS; }
    CommPollAsyncError(c, nullptr);
    *status = (HcclCommStatus)c->status.load();
    return HCCL_SUCCESS;
}
HcclResult HcclCommSuspend(HcclComm comm) { Comm *c = CommFromHandle(comm); return c ? CommSuspend(c) : HCCL_E_PTR; }
HcclResult HcclCommResume(HcclComm comm) { Comm *c = CommFromHandle(comm); return c ? CommResume(c) : HCCL_E_PTR; }
HcclResult HcclGetCommAsyncError(HcclComm comm, HcclResult *asyncError)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !asyncError) return HCCL_E_PTR;
    return CommPollAsyncError(c, asyncError);
}

HcclResult HcclCommSymAlloc(HcclComm comm, uint64_t bytes, void **ptr) { Comm *c = CommFromHandle(comm); return c ? SymAlloc(c, bytes, ptr) : HCCL_E_PTR; }
HcclResult HcclCommSetMaxCtas(HcclComm comm, uint32_t maxCtas)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    c->env.maxCtas = maxCtas;
    BumpSelectionGeneration();          // cached launch lists were planned with the old cap
    return HCCL_SUCCESS;
}
HcclResult HcclCommSymFree(HcclComm comm, void *ptr) { Comm *c = CommFromHandle(comm); return c ? SymFree(c, ptr) : HCCL_E_PTR; }
HcclResult HcclSymWinGetPeerPointer(HcclComm comm, void *localPtr, uint32_t peer, void **peerPtr)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !peerPtr) return HCCL_E_PTR;
    if (peer >= c->nranks || !SymContains(c, localPtr, 1)) return HCCL_E_PARA;
    *peerPtr = c->heap[peer] + SymOffsetOf(c, localPtr);
    return HCCL_SUCCESS;
}
HcclResult HcclSymGetMulticastPointer(HcclComm comm, void *localPtr, void **mcPtr)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !mcPtr) return HCCL_E_PTR;
    if (!c->mcHeap) return HCCL_E_UNAVAIL;
    if (!SymContains(c, localPtr, 1)) return HCCL_E_PARA;
    *mcPtr = c->mcHeap + SymOffsetOf(c, localPtr);
    return HCCL_SUCCESS;
}
HcclResult HcclSimStreamSynchronize(HcclComm comm)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (!c->worker) return HCCL_SUCCESS;
    HcclResult r = c->worker->Drain();
    if (r == HCCL_E_TIMEOUT) CommPollAsyncError(c, nullptr);
    return r;
}

}  // extern "C"
