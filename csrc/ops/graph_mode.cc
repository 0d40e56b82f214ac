#include "hccl/hccl_graph_mode.h"
#include <cstring>
#include "../exec/executor.h"
#include "../kernels/coll_args.h"
#include "../select/selector.h"
#include "hccl/hccl.h"
#include "op_entry.h"

using namespace hccl;

namespace hccl {
Comm *CommFindByName(const char *name);
}

namespace {

struct GraphParam {
    uint32_t magic = 0x47504d31u;
    HcclCMDType opType = HCCL_CMD_INVALID;
    uint64_t count = 0;
    HcclDataType dtype = HCCL_DATA_TYPE_FP32;
    HcclReduceOp op = HCCL_REDUCE_SUM;
    uint32_t root = 0;
    char group[HCCL_COMM_NAME_MAX] = {0};
};
GraphParam *GP(void *p)
{
    auto *g = static_cast<GraphParam *>(p);
    return (g && g->magic == 0x47504d31u) ? g : nullptr;
}

// Common tail of every graph-mode entry: find the communicator by group name, mark the call as offload mode.
HcclResult GraphCommon(const char *group, const char *tag, cudaStream_t *streams, uint32_t streamNum, void *scratch, uint64_t scratchSize, Comm **c, OpParam *p)
{
    CHK_RET(InitEnvConfig());
    CHK_PTR_NULL(group);
    CHK_RET(HcomCheckTag(tag));
    *c = CommFindByName(group);
    CHK_PRT_RET(*c == nullptr, HCCL_ERROR("[EI0003] graph mode: no communicator named '%s'", group), HCCL_E_NOT_FOUND);
    CHK_PRT_RET(streamNum > 0 && streams == nullptr, HCCL_ERROR("[EI0003] graph mode: %u helper streams announced but none given", streamNum), HCCL_E_PTR);
    p->mode = OpMode::OFFLOAD;
    p->tag = tag;
    for (uint32_t i = 0; i < streamNum; ++i) p->slaveStreams.push_back(streams[i]);
    p->graphScratch = scratch;
    p->graphScratchBytes = scratchSize;
    return HCCL_SUCCESS;
}

HcclResult FillFromGraphParam(const GraphParam &g, uint32_t nranks, OpParam *p)
{
    p->opType = g.opType;
    p->count = g.count;
    p->dtype = p->outDtype = g.dtype;
    p->reduceOp = g.op;
    p->root = g.root;
    p->tag = std::string(CmdName(g.opType)) + "_graph";
    if (g.opType == HCCL_CMD_ALLTOALLV || g.opType == HCCL_CMD_ALLTOALLVC || g.opType == HCCL_CMD_ALLGATHER_V || g.opType == HCCL_CMD_REDUCE_SCATTER_V) {
        p->sendCounts.assign(nranks, g.count); p->recvCounts.assign(nranks, g.count);
        p->sendDispls.resize(nranks); p->recvDispls.resize(nranks);
        for (uint32_t r = 0; r < nranks; ++r) p->sendDispls[r] = p->recvDispls[r] = r * g.count;
    }
    return g.opType == HCCL_CMD_INVALID ? HCCL_E_PARA : HCCL_SUCCESS;
}

HcclResult CalcRes(Comm *c, uint32_t nranks, uint64_t cclBytes, bool nvls, const GraphParam &g, HcclOpResGraphMode *res)
{
    memset(res, 0, sizeof(*res));
    OpParam p;
    CHK_RET(FillFromGraphParam(g, nranks, &p));
    RegisterBuiltinExecutors();
    if (c) {
        CHK_RET(SelectAlgorithm(c, p, {}));
    } else {
        // offline: the CUDA cascade without a communicator, under the current environment; an NVSwitch multicast mapping
        // is assumed to exist unless HCCL_NVLS_ENABLE=0 (the target is an 8 x B200 NVSwitch box)
        const AlgEnvConfig &env = GetEnvConfig();
        TopoInfo topo;
        CHK_RET(BuildSimTopoInfo(1, 1, nranks, 0, &topo));
        SelectorCtx ctx{nullptr, &topo, &env, true, nvls, cclBytes, {}};
        CHK_RET(ExecuteSelector(ctx, p));
    }
    snprintf(res->algName, sizeof(res->algName), "%s", p.algName.c_str());
    res->engine = (uint32_t)p.engine;
    if (p.engine == HCCL_ENGINE_SM || p.engine == HCCL_ENGINE_NVLS) {
        SmPlanCtx ctx{0, nranks, cclBytes, 2u << 20, c ? c->env.maxCtas : 0u, nvls};
        std::vector<SmLaunch> launches;
        HcclResult r = SmPlanOp(ctx, p, p.algName, &launches);
        if (r == HCCL_E_NOT_SUPPORT) {   // same fallback the dispatch core would take
            p.algName = TuningTable::Instance().Lookup(p.opType, nranks, HCCL_ENGINE_SM, p.DataBytes()) ? TuningTable::Instance().Lookup(p.opType, nranks, HCCL_ENGINE_SM, p.DataBytes())->algName : p.algName;
            snprintf(res->algName, sizeof(res->algName), "%s", p.algName.c_str());
            res->engine = HCCL_ENGINE_SM;
            launches.clear();
            r = SmPlanOp(ctx, p, p.algName, &launches);
        }
        CHK_RET(r);
        res->taskNum = (uint32_t)launches.size();
        for (auto &l : launches) res->ctaNum = std::max(res->ctaNum, l.ctas);
        res->scratchBytes = std::min<uint64_t>(cclBytes, p.DataBytes() * nranks + (1u << 20));
        res->streamNum = 0;
    } else {
        RegisterBuiltinIrTemplates();
        const IrTemplate *t = IrTemplateRegistry::Instance().Find(p.algName);
        if (t) {
            std::vector<TemplateCtx> chunks;
            CHK_RET(BuildFlatChunks(p, 0, nranks, cclBytes, *t, &chunks));
            for (auto &ctx : chunks) { Plan pl; CHK_RET(t->gen(ctx, &pl)); res->taskNum += (uint32_t)pl.TaskCount(); }
        }
        res->scratchBytes = cclBytes;
        res->streamNum = 0;
    }
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" {

#define GRAPH_ARGS group, tag, streams, streamNum, scratch, scratchSize

HcclResult HcclAllReduceGraphMode(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclAllReduceGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (count == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf); CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(count)); CHK_RET(HcomCheckReduceDataType(dataType, op));
        p.opType = HCCL_CMD_ALLREDUCE; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = count; p.dtype = p.outDtype = dataType; p.reduceOp = op;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclAllGatherGraphMode(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclAllGatherGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (sendCount == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf); CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(sendCount)); CHK_RET(HcomCheckDataType(dataType));
        p.opType = HCCL_CMD_ALLGATHER; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = sendCount; p.dtype = p.outDtype = dataType;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclReduceScatterGraphMode(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclReduceScatterGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (recvCount == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf); CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(recvCount)); CHK_RET(HcomCheckReduceDataType(dataType, op));
        p.opType = HCCL_CMD_REDUCE_SCATTER; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = recvCount; p.dtype = p.outDtype = dataType; p.reduceOp = op;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclBroadcastGraphMode(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclBroadcastGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (count == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(buf);
        CHK_RET(HcomCheckCount(count)); CHK_RET(HcomCheckDataType(dataType)); CHK_RET(HcomCheckUserRank(c->nranks, root));
        p.opType = HCCL_CMD_BROADCAST; p.stream = stream; p.inputPtr = buf; p.outputPtr = buf; p.count = count; p.dtype = p.outDtype = dataType; p.root = root;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclReduceGraphMode(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclReduceGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (count == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf);
        CHK_RET(HcomCheckUserRank(c->nranks, root));
        if (c->rank == root) CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(count)); CHK_RET(HcomCheckReduceDataType(dataType, op));
        p.opType = HCCL_CMD_REDUCE; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = count; p.dtype = p.outDtype = dataType; p.reduceOp = op; p.root = root;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclScatterGraphMode(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclScatterGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (recvCount == 0) return HCCL_SUCCESS;
        CHK_RET(HcomCheckUserRank(c->nranks, root));
        if (c->rank == root) CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(recvCount)); CHK_RET(HcomCheckDataType(dataType));
        p.opType = HCCL_CMD_SCATTER; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = recvCount; p.dtype = p.outDtype = dataType; p.root = root;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclAlltoAllGraphMode(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf, uint64_t recvCount,
                                 HcclDataType recvType, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclAlltoAllGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        if (sendCount == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf); CHK_PTR_NULL(recvBuf);
        CHK_PRT_RET(sendCount != recvCount || sendType != recvType || sendBuf == recvBuf, HCCL_ERROR("[EI0003] AlltoAll graph mode: mismatching send / receive description"), HCCL_E_PARA);
        CHK_RET(HcomCheckDataType(sendType));
        p.opType = HCCL_CMD_ALLTOALL; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = const_cast<void *>(recvBuf); p.count = sendCount; p.dtype = sendType; p.outDtype = recvType;
        return HcclExecOp(c, p);
    });
}
// The variable-count forms (reference: src/ops/all_gather_v/all_gather_v_op.h:31, src/ops/reduce_scatter_v/reduce_scatter_v_op.h:30,
// src/ops/all_to_all_v/all_to_all_v_op.h:36-41). Count and displacement arrays are host arrays of nranks uint64_t, read at the call:
// a captured graph replays the counts it was captured with.
HcclResult HcclAllGatherVGraphMode(void *sendBuf, void *recvBuf, uint64_t sendCount, const void *recvCounts, const void *recvDispls, HcclDataType dataType,
                                   HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclAllGatherVGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        CHK_PTR_NULL(recvCounts); CHK_PTR_NULL(recvDispls);
        CHK_RET(HcomCheckDataType(dataType));
        const uint64_t *rc = (const uint64_t *)recvCounts, *rd = (const uint64_t *)recvDispls;
        p.recvCounts.assign(rc, rc + c->nranks);
        p.recvDispls.assign(rd, rd + c->nranks);
        uint64_t total = 0;
        for (uint64_t v : p.recvCounts) { CHK_RET(HcomCheckCount(v)); total += v; }
        CHK_PRT_RET(p.recvCounts[c->rank] != sendCount, HCCL_ERROR("[EI0003] AllGatherV graph mode: sendCount %llu differs from recvCounts[%u] = %llu",
                    (unsigned long long)sendCount, c->rank, (unsigned long long)p.recvCounts[c->rank]), HCCL_E_PARA);
        if (total == 0) return HCCL_SUCCESS;
        if (sendCount) CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        p.opType = HCCL_CMD_ALLGATHER_V; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = sendCount; p.dtype = p.outDtype = dataType;
        return HcclExecOp(c, p);
    });
}
HcclResult HcclReduceScatterVGraphMode(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                                       HcclReduceOp op, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclReduceScatterVGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        CHK_PTR_NULL(sendCounts); CHK_PTR_NULL(sendDispls);
        CHK_PRT_RET(op == HCCL_REDUCE_PROD, HCCL_ERROR("[EI0003] ReduceScatterV supports sum, max and min only"), HCCL_E_NOT_SUPPORT);
        CHK_RET(HcomCheckReduceDataType(dataType, op));
        CHK_PRT_RET(dataType == HCCL_DATA_TYPE_UINT64 || dataType == HCCL_DATA_TYPE_FP64, HCCL_ERROR("[EI0003] ReduceScatterV does not support %s", DataTypeName(dataType)),
                    HCCL_E_NOT_SUPPORT);
        const uint64_t *sc = (const uint64_t *)sendCounts, *sd = (const uint64_t *)sendDispls;
        p.sendCounts.assign(sc, sc + c->nranks);
        p.sendDispls.assign(sd, sd + c->nranks);
        uint64_t total = 0;
        for (uint64_t v : p.sendCounts) { CHK_RET(HcomCheckCount(v)); total += v; }
        CHK_PRT_RET(p.sendCounts[c->rank] != recvCount, HCCL_ERROR("[EI0003] ReduceScatterV graph mode: recvCount %llu differs from sendCounts[%u] = %llu",
                    (unsigned long long)recvCount, c->rank, (unsigned long long)p.sendCounts[c->rank]), HCCL_E_PARA);
        if (total == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf);
        if (recvCount) CHK_PTR_NULL(recvBuf);
        p.opType = HCCL_CMD_REDUCE_SCATTER_V; p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = recvCount; p.dtype = p.outDtype = dataType; p.reduceOp = op;
        return HcclExecOp(c, p);
    });
}
static HcclResult AlltoAllVGraph(Comm *c, OpParam &p, const void *sendBuf, const void *recvBuf, cudaStream_t stream)
{
    uint64_t totalSend = 0, totalRecv = 0;
    for (uint32_t r = 0; r < c->nranks; ++r) {
        CHK_RET(HcomCheckCount(p.sendCounts[r])); CHK_RET(HcomCheckCount(p.recvCounts[r]));
        totalSend += p.sendCounts[r]; totalRecv += p.recvCounts[r];
    }
    CHK_PRT_RET(p.sendCounts[c->rank] * DataTypeSize(p.dtype) != p.recvCounts[c->rank] * DataTypeSize(p.outDtype),
                HCCL_ERROR("[EI0003] AlltoAllV graph mode: the block a rank sends to itself must equal the block it receives from itself"), HCCL_E_PARA);
    if (totalSend) CHK_PTR_NULL(sendBuf);
    if (totalRecv) CHK_PTR_NULL(recvBuf);
    CHK_PRT_RET(sendBuf != nullptr && sendBuf == recvBuf, HCCL_ERROR("[EI0003] AlltoAllV graph mode: sendBuf and recvBuf must differ"), HCCL_E_PARA);
    p.stream = stream; p.inputPtr = sendBuf; p.outputPtr = const_cast<void *>(recvBuf);
    return HcclExecOp(c, p);       // ranks without data still take part: the others wait for them
}
HcclResult HcclAlltoAllVGraphMode(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType, const void *recvBuf,
                                  const void *recvCounts, const void *rdispls, HcclDataType recvType, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclAlltoAllVGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        CHK_PTR_NULL(sendCounts); CHK_PTR_NULL(sdispls); CHK_PTR_NULL(recvCounts); CHK_PTR_NULL(rdispls);
        CHK_RET(HcomCheckDataType(sendType)); CHK_RET(HcomCheckDataType(recvType));
        const uint32_t n = c->nranks;
        p.sendCounts.assign((const uint64_t *)sendCounts, (const uint64_t *)sendCounts + n);
        p.sendDispls.assign((const uint64_t *)sdispls, (const uint64_t *)sdispls + n);
        p.recvCounts.assign((const uint64_t *)recvCounts, (const uint64_t *)recvCounts + n);
        p.recvDispls.assign((const uint64_t *)rdispls, (const uint64_t *)rdispls + n);
        p.opType = HCCL_CMD_ALLTOALLV; p.dtype = sendType; p.outDtype = recvType;
        return AlltoAllVGraph(c, p, sendBuf, recvBuf, stream);
    });
}
HcclResult HcclAlltoAllVCGraphMode(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf, HcclDataType recvType,
                                   HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclAlltoAllVCGraphMode", [&]() -> HcclResult {
        Comm *c; OpParam p;
        CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
        CHK_PTR_NULL(sendCountMatrix);
        CHK_RET(HcomCheckDataType(sendType)); CHK_RET(HcomCheckDataType(recvType));
        CHK_PRT_RET(DataTypeSize(sendType) != DataTypeSize(recvType), HCCL_ERROR("[EI0003] AlltoAllVC graph mode: send and receive element sizes differ"), HCCL_E_PARA);
        const uint32_t n = c->nranks, me = c->rank;
        const uint64_t *M = (const uint64_t *)sendCountMatrix;
        p.sendCounts.resize(n); p.sendDispls.resize(n); p.recvCounts.resize(n); p.recvDispls.resize(n);
        uint64_t so = 0, ro = 0;
        for (uint32_t j = 0; j < n; ++j) {
            p.sendCounts[j] = M[(uint64_t)me * n + j]; p.sendDispls[j] = so; so += p.sendCounts[j];
            p.recvCounts[j] = M[(uint64_t)j * n + me]; p.recvDispls[j] = ro; ro += p.recvCounts[j];
        }
        p.opType = HCCL_CMD_ALLTOALLVC; p.dtype = sendType; p.outDtype = recvType;
        return AlltoAllVGraph(c, p, sendBuf, recvBuf, stream);
    });
}
static HcclResult P2pGraph(HcclCMDType op, void *buf, uint64_t count, HcclDataType dataType, uint32_t peer, HCCL_GRAPH_MODE_TAIL)
{
    Comm *c; OpParam p;
    CHK_RET(GraphCommon(GRAPH_ARGS, &c, &p));
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(buf);
    CHK_RET(HcomCheckCount(count)); CHK_RET(HcomCheckDataType(dataType)); CHK_RET(HcomCheckUserRank(c->nranks, peer));
    CHK_PRT_RET(peer == c->rank, HCCL_ERROR("[EI0003] graph mode p2p: peer equals own rank"), HCCL_E_PARA);
    p.opType = op; p.stream = stream; p.inputPtr = buf; p.outputPtr = buf; p.count = count; p.dtype = p.outDtype = dataType; p.peer = peer;
    return HcclExecOp(c, p);
}
HcclResult HcclSendGraphMode(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclSendGraphMode", [&] { return P2pGraph(HCCL_CMD_SEND, sendBuf, count, dataType, destRank, group, stream, tag, streams, streamNum, scratch, scratchSize); });
}
HcclResult HcclRecvGraphMode(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HCCL_GRAPH_MODE_TAIL)
{
    return Guard("HcclRecvGraphMode", [&] { return P2pGraph(HCCL_CMD_RECEIVE, recvBuf, count, dataType, srcRank, group, stream, tag, streams, streamNum, scratch, scratchSize); });
}

HcclResult HcclOpParamGraphModeCreate(HcclOpParamGraphMode *param)
{
    CHK_PTR_NULL(param);
    *param = new (std::nothrow) GraphParam();
    return *param ? HCCL_SUCCESS : HCCL_E_MEMORY;
}
HcclResult HcclOpParamGraphModeDestroy(HcclOpParamGraphMode param)
{
    GraphParam *g = GP(param);
    if (!g) return HCCL_E_PTR;
    g->magic = 0;
    delete g;
    return HCCL_SUCCESS;
}
#define GP_SET(name, type, field, check)                                           \
    HcclResult HcclOpParamGraphModeSet##name(HcclOpParamGraphMode param, type v)  \
    {                                                                              \
        GraphParam *g = GP(param);                                                 \
        if (!g) return HCCL_E_PTR;                                                 \
        check;                                                                     \
        g->field = v;                                                              \
        return HCCL_SUCCESS;                                                       \
    }
GP_SET(OpType, HcclCMDType, opType, if (v == HCCL_CMD_INVALID || v >= HCCL_CMD_MAX) return HCCL_E_PARA)
GP_SET(DataCount, uint64_t, count, CHK_RET(HcomCheckCount(v)))
GP_SET(DataType, HcclDataType, dtype, CHK_RET(HcomCheckDataType(v)))
GP_SET(ReduceOp, HcclReduceOp, op, CHK_RET(HcomCheckReductionOp(v)))
GP_SET(Root, uint32_t, root, (void)0)
HcclResult HcclOpParamGraphModeSetGroup(HcclOpParamGraphMode param, const char *group)
{
    GraphParam *g = GP(param);
    if (!g || !group) return HCCL_E_PTR;
    if (strnlen(group, HCCL_COMM_NAME_MAX) >= HCCL_COMM_NAME_MAX) return HCCL_E_PARA;
    snprintf(g->group, sizeof(g->group), "%s", group);
    return HCCL_SUCCESS;
}

HcclResult HcclCalcOpResOfflineGraphMode(HcclOpParamGraphMode param, uint32_t rankSize, HcclOpResGraphMode *res)
{
    GraphParam *g = GP(param);
    if (!g || !res) return HCCL_E_PTR;
    if (rankSize < 2 || rankSize > (uint32_t)kMaxRanks) return HCCL_E_PARA;
    InitEnvConfig();
    return Guard("HcclCalcOpResOfflineGraphMode", [&] { return CalcRes(nullptr, rankSize, GetEnvConfig().bufferSizeBytes, GetEnvConfig().nvlsEnable, *g, res); });
}
HcclResult HcclCalcOpResOnlineGraphMode(HcclComm comm, HcclOpParamGraphMode param, HcclOpResGraphMode *res)
{
    GraphParam *g = GP(param);
    if (!g || !res) return HCCL_E_PTR;
    Comm *c = comm ? CommFromHandle(comm) : CommFindByName(g->group);
    if (!c) return HCCL_E_NOT_FOUND;
    if (c->nranks < 2) { memset(res, 0, sizeof(*res)); snprintf(res->algName, sizeof(res->algName), "SingleRank"); return HCCL_SUCCESS; }
    return Guard("HcclCalcOpResOnlineGraphMode", [&] { return CalcRes(c, c->nranks, c->devComm.cclBytes, c->mcHeap != nullptr, *g, res); });
}
HcclResult HcclSelectAlgGraphMode(HcclComm comm, HcclOpParamGraphMode param, char *algName, uint32_t algNameLen)
{
    HcclOpResGraphMode res;
    CHK_RET(HcclCalcOpResOnlineGraphMode(comm, param, &res));
    if (!algName || algNameLen == 0) return HCCL_E_PTR;
    snprintf(algName, algNameLen, "%s", res.algName);
    return HCCL_SUCCESS;
}

}  // extern "C"
