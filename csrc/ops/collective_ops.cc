// Collective operator entries: AllReduce, Broadcast, ReduceScatter(V), Scatter, AllGather(V), Reduce, Barrier.
// Reference entries: src/ops/all_reduce/all_reduce_op.cc:23, broadcast/broadcast_op.cc:23,
// reduce_scatter/reduce_scatter_op.cc:23, reduce_scatter_v/reduce_scatter_v_op.cc:24, scatter/scatter_op.cc:30,
// all_gather/all_gather_op.cc:24, all_gather_v/all_gather_v_op.cc:22, reduce/reduce_op.cc:23, barrier/barrier_op.cc:44.
#include "hccl/hccl.h"
#include "op_entry.h"

using namespace hccl;

extern "C" {

HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                         cudaStream_t stream)
{
    return Guard("HcclAllReduce", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (count == 0) { HCCL_WARNING("HcclAllReduce: count is 0, nothing to do"); return HCCL_SUCCESS; }
        CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(count));
        CHK_RET(HcomCheckReduceDataType(dataType, op));
        OpParam p = MakeParam(c, HCCL_CMD_ALLREDUCE, "AllReduce", stream);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = count; p.dtype = p.outDtype = dataType; p.reduceOp = op;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclBroadcast", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (count == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(buf);
        CHK_RET(HcomCheckCount(count));
        CHK_RET(HcomCheckDataType(dataType));
        CHK_RET(HcomCheckUserRank(c->nranks, root));
        OpParam p = MakeParam(c, HCCL_CMD_BROADCAST, "Broadcast", stream);
        p.inputPtr = buf; p.outputPtr = buf; p.count = count; p.dtype = p.outDtype = dataType; p.root = root;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                             cudaStream_t stream)
{
    return Guard("HcclReduceScatter", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (recvCount == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(recvCount));
        CHK_RET(HcomCheckCount(recvCount * c->nranks));
        CHK_RET(HcomCheckReduceDataType(dataType, op));
        OpParam p = MakeParam(c, HCCL_CMD_REDUCE_SCATTER, "ReduceScatter", stream);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = recvCount; p.dtype = p.outDtype = dataType; p.reduceOp = op;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclReduceScatterV(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf, uint64_t recvCount,
                              HcclDataType dataType, HcclReduceOp op, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclReduceScatterV", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        CHK_PTR_NULL(sendCounts);
        CHK_PTR_NULL(sendDispls);
        if (op == HCCL_REDUCE_PROD) { HCCL_ERROR("[EI0003] ReduceScatterV supports sum, max and min only"); return HCCL_E_NOT_SUPPORT; }
        CHK_RET(HcomCheckReduceDataType(dataType, op));
        if (dataType == HCCL_DATA_TYPE_UINT64 || dataType == HCCL_DATA_TYPE_FP64) { HCCL_ERROR("[EI0003] ReduceScatterV does not support %s", DataTypeName(dataType)); return HCCL_E_NOT_SUPPORT; }
        OpParam p = MakeParam(c, HCCL_CMD_REDUCE_SCATTER_V, "ReduceScatterV", stream);
        const uint64_t *sc = (const uint64_t *)sendCounts, *sd = (const uint64_t *)sendDispls;
        p.sendCounts.assign(sc, sc + c->nranks);
        p.sendDispls.assign(sd, sd + c->nranks);
        uint64_t total = 0;
        for (uint64_t v : p.sendCounts) { CHK_RET(HcomCheckCount(v)); total += v; }
        if (p.sendCounts[c->rank] != recvCount) {
            HCCL_ERROR("[EI0003] ReduceScatterV: recvCount %llu differs from sendCounts[%u] = %llu", (unsigned long long)recvCount, c->rank,
                       (unsigned long long)p.sendCounts[c->rank]);
            return HCCL_E_PARA;
        }
        if (total == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf);
        if (recvCount) CHK_PTR_NULL(recvBuf);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = recvCount; p.dtype = p.outDtype = dataType; p.reduceOp = op;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, HcclComm comm,
                       cudaStream_t stream)
{
    return Guard("HcclScatter", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (recvCount == 0) return HCCL_SUCCESS;
        CHK_RET(HcomCheckUserRank(c->nranks, root));
        if (c->rank == root) CHK_PTR_NULL(sendBuf);   // only the root needs a send buffer
        CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(recvCount));
        CHK_RET(HcomCheckDataType(dataType));
        OpParam p = MakeParam(c, HCCL_CMD_SCATTER, "Scatter", stream);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = recvCount; p.dtype = p.outDtype = dataType; p.root = root;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclAllGather", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (sendCount == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(sendCount));
        CHK_RET(HcomCheckCount(sendCount * c->nranks));
        CHK_RET(HcomCheckDataType(dataType));
        OpParam p = MakeParam(c, HCCL_CMD_ALLGATHER, "AllGather", stream);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = sendCount; p.dtype = p.outDtype = dataType;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclAllGatherV(void *sendBuf, uint64_t sendCount, void *recvBuf, const void *recvCounts, const void *recvDispls,
                          HcclDataType dataType, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclAllGatherV", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        CHK_PTR_NULL(recvCounts);
        CHK_PTR_NULL(recvDispls);
        CHK_RET(HcomCheckDataType(dataType));
        OpParam p = MakeParam(c, HCCL_CMD_ALLGATHER_V, "AllGatherV", stream);
        const uint64_t *rc = (const uint64_t *)recvCounts, *rd = (const uint64_t *)recvDispls;
        p.recvCounts.assign(rc, rc + c->nranks);
        p.recvDispls.assign(rd, rd + c->nranks);
        uint64_t total = 0;
        for (uint64_t v : p.recvCounts) { CHK_RET(HcomCheckCount(v)); total += v; }
        if (p.recvCounts[c->rank] != sendCount) {
            HCCL_ERROR("[EI0003] AllGatherV: sendCount %llu differs from recvCounts[%u] = %llu", (unsigned long long)sendCount, c->rank,
                       (unsigned long long)p.recvCounts[c->rank]);
            return HCCL_E_PARA;
        }
        if (total == 0) return HCCL_SUCCESS;
        if (sendCount) CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = sendCount; p.dtype = p.outDtype = dataType;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, HcclComm comm,
                      cudaStream_t stream)
{
    return Guard("HcclReduce", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (count == 0) return HCCL_SUCCESS;
        CHK_RET(HcomCheckUserRank(c->nranks, root));
        CHK_PTR_NULL(sendBuf);
        if (c->rank == root) CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckCount(count));
        CHK_RET(HcomCheckReduceDataType(dataType, op));
        OpParam p = MakeParam(c, HCCL_CMD_REDUCE, "Reduce", stream);
        p.inputPtr = sendBuf; p.outputPtr = recvBuf; p.count = count; p.dtype = p.outDtype = dataType; p.reduceOp = op; p.root = root;
        return HcclExecOp(c, p);
    });
}

HcclResult HcclBarrier(HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclBarrier", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (c->nranks == 1) return HCCL_SUCCESS;
        OpParam p = MakeParam(c, HCCL_CMD_BARRIER, "Barrier", stream);
        p.dtype = p.outDtype = HCCL_DATA_TYPE_INT8;
        return HcclExecOp(c, p);
    });
}

}  // extern "C"
