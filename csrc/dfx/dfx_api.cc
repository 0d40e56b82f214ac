#include <cstring>
#include <fstream>
#include <sstream>
#include "../common/dtype.h"
#include "../common/env_config.h"
#include "../common/log.h"
#include "../core/comm.h"
#include "../exec/executor.h"
#include "../exec/op_common.h"
#include "../select/selector.h"
#include "hccl/hccl_dfx.h"

using namespace hccl;

static HcclResult CopyOut(const std::string &s, char *buf, uint32_t len)
{
    if (!buf || len == 0) return HCCL_E_PTR;
    snprintf(buf, len, "%s", s.c_str());
    return s.size() < len ? HCCL_SUCCESS : HCCL_E_MEMORY;
}

extern "C" {

int HcclCommIsCuda(HcclComm comm) { Comm *c = CommFromHandle(comm); return c && c->backend == BackendKind::CUDA; }
int HcclCommHasNvls(HcclComm comm) { Comm *c = CommFromHandle(comm); return c && c->mcHeap != nullptr; }

HcclResult HcclGetCommCounters(HcclComm comm, HcclCommCounters *out)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !out) return HCCL_E_PTR;
    out->ops = c->counters.ops; out->bytes = c->counters.bytes; out->timeouts = c->counters.timeouts;
    out->planCacheHits = c->counters.planCacheHits; out->planCacheMisses = c->counters.planCacheMisses;
    out->fallbacks = c->counters.fallbacks; out->consistencyChecks = c->counters.consistencyChecks;
    out->chunkLoops = c->counters.chunkLoops; out->kernelsLaunched = c->counters.kernelsLaunched;
    return HCCL_SUCCESS;
}

HcclResult HcclGetLastOps(HcclComm comm, HcclOpRecordC *out, uint32_t maxRecords, uint32_t *numRecords)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !out || !numRecords) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(c->opRingMu);
    uint32_t n = 0;
    size_t start = c->opRing.size() > maxRecords ? c->opRing.size() - maxRecords : 0;
    for (size_t i = start; i < c->opRing.size(); ++i, ++n) {
        const OpRecord &r = c->opRing[i];
        HcclOpRecordC &o = out[n];
        memset(&o, 0, sizeof(o));
        o.seq = r.seq; o.opType = r.opType; o.dataType = r.dtype; o.reduceOp = r.reduceOp; o.root = r.root; o.engine = r.engine;
        o.count = r.count; o.beginNs = r.beginNs; o.endNs = r.endNs;
        memcpy(o.algName, r.algName, sizeof(o.algName));
    }
    *numRecords = n;
    return HCCL_SUCCESS;
}

HcclResult HcclGetAlgoHistogram(HcclComm comm, char *buf, uint32_t bufLen)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    std::ostringstream os;
    std::lock_guard<std::mutex> lk(c->counters.mu);
    for (auto &kv : c->counters.algoHistogram) os << kv.first << "=" << kv.second << ";";
    return CopyOut(os.str(), buf, bufLen);
}

HcclResult HcclQuerySelection(HcclComm comm, HcclCMDType op, uint64_t count, HcclDataType dataType, HcclReduceOp reduceOp, char *algName,
                              uint32_t algNameLen, uint32_t *engine)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    RegisterBuiltinExecutors();
    OpParam p;
    p.opType = op; p.count = count; p.dtype = p.outDtype = dataType; p.reduceOp = reduceOp; p.tag = std::string(CmdName(op)) + "_" + c->name;
    if (op == HCCL_CMD_ALLTOALLV || op == HCCL_CMD_ALLTOALLVC || op == HCCL_CMD_ALLGATHER_V || op == HCCL_CMD_REDUCE_SCATTER_V) {
        p.sendCounts.assign(c->nranks, count); p.recvCounts.assign(c->nranks, count);
        p.sendDispls.assign(c->nranks, 0); p.recvDispls.assign(c->nranks, 0);
    }
    CHK_RET(SelectAlgorithm(c, p, {}));
    if (engine) *engine = (uint32_t)p.engine;
    return CopyOut(p.algName, algName, algNameLen);
}

HcclResult HcclGetTopoDescription(HcclComm comm, char *buf, uint32_t bufLen)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    return CopyOut(c->topo.Describe(), buf, bufLen);
}

HcclResult HcclDumpTrace(HcclComm comm, const char *path)
{
    Comm *c = CommFromHandle(comm);
    if (!c || !path) return HCCL_E_PTR;
    std::ofstream f(path);
    if (!f) return HCCL_E_OPEN_FILE_FAILURE;
    f << "{\"traceEvents\":[";
    std::lock_guard<std::mutex> lk(c->opRingMu);
    bool first = true;
    for (const OpRecord &r : c->opRing) {
        if (!first) f << ",";
        first = false;
        f << "{\"name\":\"" << CmdName(r.opType) << "\",\"cat\":\"" << r.algName << "\",\"ph\":\"X\",\"pid\":" << c->rank << ",\"tid\":0,\"ts\":"
          << r.beginNs / 1000.0 << ",\"dur\":" << (r.endNs - r.beginNs) / 1000.0 << ",\"args\":{\"count\":" << r.count << ",\"dtype\":\""
          << DataTypeName(r.dtype) << "\",\"engine\":\"" << EngineName((HcclCommEngine)r.engine) << "\",\"seq\":" << r.seq << "}}";
    }
    f << "]}\n";
    return HCCL_SUCCESS;
}

void HcclSetLogLevel(int level) { LogSetLevel(level); }
uint64_t HcclGetLogRecordCount(int level) { return LogRecordCount(level); }

HcclResult HcclTuningTableLoadText(const char *text) { return text ? TuningTable::Instance().LoadText(text) : HCCL_E_PTR; }
HcclResult HcclTuningTableReset(void) { TuningTable::Instance().ResetToBuiltin(); return HCCL_SUCCESS; }
HcclResult HcclTuningTableDump(char *buf, uint32_t bufLen) { return CopyOut(TuningTable::Instance().Dump(), buf, bufLen); }

HcclResult HcclListAlgorithms(HcclCMDType op, char *buf, uint32_t bufLen)
{
    RegisterBuiltinExecutors();
    std::string s;
    for (auto &n : ExecutorRegistry::Instance().Names(op)) s += n + ";";
    return CopyOut(s, buf, bufLen);
}

void HcclResetEnvConfigForTest(void) { ResetAlgEnvConfigInitState(); }

HcclResult HcclInjectBootstrapDrop(HcclComm comm, int n)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    c->boot->InjectDropNext(n);
    return HCCL_SUCCESS;
}

}  // extern "C"
