// Send / Recv / BatchSendRecv entries (reference: src/ops/send/send_op.cc:48, src/ops/recv/recv_op.cc:46,
// src/ops/batch_send_recv/batch_send_recv_op.cc:23,90-145).
#include "hccl/hccl.h"
#include "op_entry.h"

using namespace hccl;

extern "C" {

static HcclResult P2pCommon(const char *name, HcclCMDType op, void *buf, uint64_t count, HcclDataType dataType, uint32_t peer, HcclComm comm,
                            cudaStream_t stream)
{
    Comm *c;
    CHK_RET(EntryCommon(comm, &c));
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(buf);
    CHK_RET(HcomCheckCount(count));
    CHK_RET(HcomCheckDataType(dataType));
    if (c->nranks > 1) {
        CHK_RET(HcomCheckUserRank(c->nranks, peer));
        if (peer == c->rank) { HCCL_ERROR("[EI0003] %s: peer rank equals own rank %u (use BatchSendRecv for self pairs)", name, peer); return HCCL_E_PARA; }
    }
    OpParam p = MakeParam(c, op, name, stream);
    p.inputPtr = buf; p.outputPtr = buf; p.count = count; p.dtype = p.outDtype = dataType; p.peer = peer;
    return HcclExecOp(c, p);
}

HcclResult HcclSend(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclSend", [&] { return P2pCommon("Send", HCCL_CMD_SEND, sendBuf, count, dataType, destRank, comm, stream); });
}

HcclResult HcclRecv(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclRecv", [&] { return P2pCommon("Recv", HCCL_CMD_RECEIVE, recvBuf, count, dataType, srcRank, comm, stream); });
}

HcclResult HcclBatchSendRecv(HcclSendRecvItem *sendRecvInfo, uint32_t itemNum, HcclComm comm, cudaStream_t stream)
{
    return Guard("HcclBatchSendRecv", [&]() -> HcclResult {
        Comm *c;
        CHK_RET(EntryCommon(comm, &c));
        if (itemNum == 0) return HCCL_SUCCESS;
        CHK_PTR_NULL(sendRecvInfo);
        OpParam p = MakeParam(c, HCCL_CMD_BATCH_SEND_RECV, "BatchSendRecv", stream);
        for (uint32_t i = 0; i < itemNum; ++i) {
            const HcclSendRecvItem &it = sendRecvInfo[i];
            if (it.sendRecvType != HCCL_SEND && it.sendRecvType != HCCL_RECV) { HCCL_ERROR("[EI0003] BatchSendRecv item %u: bad type %d", i, (int)it.sendRecvType); return HCCL_E_PARA; }
            CHK_RET(HcomCheckUserRank(c->nranks, it.remoteRank));
            CHK_RET(HcomCheckCount(it.count));
            CHK_RET(HcomCheckDataType(it.dataType));
            if (it.count == 0) continue;
            CHK_PTR_NULL(it.buf);
            p.items.push_back(it);
        }
        if (p.items.empty()) return HCCL_SUCCESS;
        p.dtype = p.outDtype = p.items[0].dataType;
        return HcclExecOp(c, p);
    });
}

}  // extern "C"
