/*
 * hccl_graph_mode.h -- graph (offload) mode entry points and compile-time resource queries.
 *
 * HCCL's graph engines call Hccl<Op>GraphMode with the group name, a tag, caller-provided helper streams and scratch, and
 * ask beforehand how much scratch / how many streams and tasks an operator will need (reference:
 * src/ops/all_reduce/all_reduce_op.cc:58-103; src/ops/interface_graph_mode/calc_resource_graph_mode.h:19-37 and .cc:47-94
 * with its opaque OpParamGraphMode builder). On CUDA the same calls are what a framework uses while capturing a CUDA
 * graph: all synchronisation state of this library is device-resident, so captured operators replay correctly; the
 * cross-rank consistency exchange (a host rendezvous) is skipped in this mode.
 */
#ifndef HCCL_B200_GRAPH_MODE_H_
#define HCCL_B200_GRAPH_MODE_H_

#include "hccl_comm.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_GRAPH_MODE_TAIL const char *group, cudaStream_t stream, const char *tag, cudaStream_t *streams, uint32_t streamNum, void *scratch, uint64_t scratchSize

HcclResult HcclAllReduceGraphMode(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclAllGatherGraphMode(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclReduceScatterGraphMode(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclBroadcastGraphMode(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclReduceGraphMode(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclScatterGraphMode(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclAlltoAllGraphMode(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf, uint64_t recvCount,
                                 HcclDataType recvType, HCCL_GRAPH_MODE_TAIL);
/* Variable-count forms: the count / displacement arrays are host arrays of nranks uint64_t (the matrix: nranks x nranks), read at the call. */
HcclResult HcclAllGatherVGraphMode(void *sendBuf, void *recvBuf, uint64_t sendCount, const void *recvCounts, const void *recvDispls, HcclDataType dataType,
                                   HCCL_GRAPH_MODE_TAIL);
HcclResult HcclReduceScatterVGraphMode(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                                       HcclReduceOp op, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclAlltoAllVGraphMode(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType, const void *recvBuf,
                                  const void *recvCounts, const void *rdispls, HcclDataType recvType, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclAlltoAllVCGraphMode(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf, HcclDataType recvType,
                                   HCCL_GRAPH_MODE_TAIL);
HcclResult HcclSendGraphMode(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HCCL_GRAPH_MODE_TAIL);
HcclResult HcclRecvGraphMode(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HCCL_GRAPH_MODE_TAIL);

/* Opaque operator description for the resource queries. */
typedef void *HcclOpParamGraphMode;
HcclResult HcclOpParamGraphModeCreate(HcclOpParamGraphMode *param);
HcclResult HcclOpParamGraphModeDestroy(HcclOpParamGraphMode param);
HcclResult HcclOpParamGraphModeSetOpType(HcclOpParamGraphMode param, HcclCMDType opType);
HcclResult HcclOpParamGraphModeSetDataCount(HcclOpParamGraphMode param, uint64_t count);
HcclResult HcclOpParamGraphModeSetDataType(HcclOpParamGraphMode param, HcclDataType dataType);
HcclResult HcclOpParamGraphModeSetReduceOp(HcclOpParamGraphMode param, HcclReduceOp op);
HcclResult HcclOpParamGraphModeSetRoot(HcclOpParamGraphMode param, uint32_t root);
HcclResult HcclOpParamGraphModeSetGroup(HcclOpParamGraphMode param, const char *group);

typedef struct HcclOpResGraphModeDef {
    uint64_t scratchBytes;   /* symmetric scratch the operator cycles through per chunk */
    uint32_t streamNum;      /* helper streams (0: everything runs on the caller's stream) */
    uint32_t taskNum;        /* kernel launches / schedule tasks */
    uint32_t ctaNum;         /* CTAs of the largest launch */
    char algName[128];
    uint32_t engine;
} HcclOpResGraphMode;

/* Without a communicator: estimate for `rankSize` ranks on an NVSwitch box under the current environment (buffer size, engine
 * and algorithm overrides; NVLS assumed unless HCCL_NVLS_ENABLE=0). */
HcclResult HcclCalcOpResOfflineGraphMode(HcclOpParamGraphMode param, uint32_t rankSize, HcclOpResGraphMode *res);
/* With the communicator named by the param's group (or `comm` if non-NULL): what would actually run. */
HcclResult HcclCalcOpResOnlineGraphMode(HcclComm comm, HcclOpParamGraphMode param, HcclOpResGraphMode *res);
HcclResult HcclSelectAlgGraphMode(HcclComm comm, HcclOpParamGraphMode param, char *algName, uint32_t algNameLen);

#ifdef __cplusplus
}
#endif
#endif
