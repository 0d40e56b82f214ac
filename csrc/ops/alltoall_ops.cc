// AlltoAll / AlltoAllV / AlltoAllVC entries (reference: src/ops/all_to_all_v/all_to_all_v_op.cc:23,84,144; the VC ->
// V conversion :396-430; the host count arrays are copied into the OpParam :546-611).
#include "hccl/hccl.h"
#include "op_entry.h"

using namespace hccl;

extern "C" {

HcclResult HcclAlltoAll(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf, uint64_t recvCount,
                        HcclDataType recvType, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclAlltoAll", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (sendCount == 0 && recvCount == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendBuf);
        CHK_PTR_NULL(recvBuf);
        CHK_RET(HcomCheckDataType(sendType));
        CHK_RET(HcomCheckDataType(recvType));
        if (sendCount != recvCount || sendType != recvType) {
            HCCL_ERROR("[EI0003] AlltoAll: send (%llu x %s) and receive (%llu x %s) must match", (unsigned long long)sendCount, DataTypeName(sendType),
                       (unsigned long long)recvCount, DataTypeName(recvType));
            return HCCL_E_PARA;
        }
        if (sendBuf == recvBuf) { HCCL_ERROR("[EI0003] AlltoAll: sendBuf and recvBuf must differ"); return HCCL_E_PARA; }
        CHK_RET(HcomCheckCount(sendCount * c->nranks));
        OpParam p = MakeParam(c, HCCL_CMD_ALLTOALL, "AlltoAll", stream);
        p.inputPtr = sendBuf; p.outputPtr = const_cast<void *>(recvBuf); p.count = sendCount; p.dtype = sendType; p.outDtype = recvType;
        return HcclExecOp(c, p);
    });
}

static HcclResult AlltoAllVCommon(Comm *c, OpParam &p, const void *sendBuf, const void *recvBuf)
{
    uint64_t totalSend = 0, totalRecv = 0;
    for (uint32_t r = 0; r < c->nranks; ++r) {
        CHK_RET(HcomCheckCount(p.sendCounts[r]));
        CHK_RET(HcomCheckCount(p.recvCounts[r]));
        totalSend += p.sendCounts[r];
        totalRecv += p.recvCounts[r];
    }
    if (p.sendCounts[c->rank] * DataTypeSize(p.dtype) != p.recvCounts[c->rank] * DataTypeSize(p.outDtype)) {
        HCCL_ERROR("[EI0003] AlltoAllV: the block a rank sends to itself must equal the block it receives from itself");
        return HCCL_E_PARA;
    }
    if (totalSend == 0 && totalRecv == 0) {
        // still a synchronising call for the others? No: every rank sees zero in its own row/column only. Run the
        // exchange so ranks with data are not left waiting on this one.
    }
    if (totalSend) CHK_PTR_NULL(sendBuf);
    if (totalRecv) CHK_PTR_NULL(recvBuf);
    if (sendBuf != nullptr && sendBuf == recvBuf) { HCCL_ERROR("[EI0003] AlltoAllV: sendBuf and recvBuf must differ"); return HCCL_E_PARA; }
    p.inputPtr = sendBuf;
    p.outputPtr = const_cast<void *>(recvBuf);
    return HcclExecOp(c, p);
}

HcclResult HcclAlltoAllV(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType, const void *recvBuf,
                         const void *recvCounts, const void *rdispls, HcclDataType recvType, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclAlltoAllV", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        CHK_PTR_NULL(sendCounts);
        CHK_PTR_NULL(sdispls);
        CHK_PTR_NULL(recvCounts);
        CHK_PTR_NULL(rdispls);
        CHK_RET(HcomCheckDataType(sendType));
        CHK_RET(HcomCheckDataType(recvType));
        OpParam p = MakeParam(c, HCCL_CMD_ALLTOALLV, "AlltoAllV", stream);
        uint32_t n = c->nranks;
        p.sendCounts.assign((const uint64_t *)sendCounts, (const uint64_t *)sendCounts + n);
        p.sendDispls.assign((const uint64_t *)sdispls, (const uint64_t *)sdispls + n);
        p.recvCounts.assign((const uint64_t *)recvCounts, (const uint64_t *)recvCounts + n);
        p.recvDispls.assign((const uint64_t *)rdispls, (const uint64_t *)rdispls + n);
        p.dtype = sendType; p.outDtype = recvType;
        return AlltoAllVCommon(c, p, sendBuf, recvBuf);
    });
}

// The count matrix M[i][j] (elements rank i sends to rank j) is known to every rank; rows are packed contiguously in
// the send buffer and columns in the receive buffer, which yields the V form.
HcclResult HcclAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf, HcclDataType recvType,
                          HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclAlltoAllVC", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        CHK_PTR_NULL(sendCountMatrix);
        CHK_RET(HcomCheckDataType(sendType));
        CHK_RET(HcomCheckDataType(recvType));
        if (DataTypeSize(sendType) != DataTypeSize(recvType)) { HCCL_ERROR("[EI0003] AlltoAllVC: send and receive element sizes differ"); return HCCL_E_PARA; }
        OpParam p = MakeParam(c, HCCL_CMD_ALLTOALLVC, "AlltoAllVC", stream);
        uint32_t n = c->nranks, me = c->rank;
        const uint64_t *M = (const uint64_t *)sendCountMatrix;
        p.sendCounts.resize(n); p.sendDispls.resize(n); p.recvCounts.resize(n); p.recvDispls.resize(n);
        uint64_t so = 0, ro = 0;
        for (uint32_t j = 0; j < n; ++j) {
            p.sendCounts[j] = M[(uint64_t)me * n + j]; p.sendDispls[j] = so; so += p.sendCounts[j];
            p.recvCounts[j] = M[(uint64_t)j * n + me]; p.recvDispls[j] = ro; ro += p.recvCounts[j];
        }
        p.dtype = sendType; p.outDtype = recvType;
        return AlltoAllVCommon(c, p, sendBuf, recvBuf);
    });
}

}  // extern "C"
