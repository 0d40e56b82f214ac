/*
 * hccl.h -- collective and point-to-point operators.
 *
 * Same entry points, argument order and semantics as HCCL's public header (reference:
 * include/hccl.h:35-249) plus HcclBarrier (reference: src/ops/barrier/barrier_op.cc:44); the stream
 * argument is a cudaStream_t. With the host simulation backend the stream argument is ignored and
 * ops run on the communicator's worker queue.
 *
 * Counts are in elements. Reduction dtypes: int8/16/32/64, uint64, fp16, fp32, fp64, bf16.
 * PROD is limited to int8/int32/int64/uint64/fp16/fp32/fp64. count == 0 succeeds without work.
 */
#ifndef HCCL_B200_H_
#define HCCL_B200_H_

#include "hccl_types.h"
#include "hccl_comm.h"

#ifdef __cplusplus
extern "C" {
#endif

HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                         HcclComm comm, cudaStream_t stream);
HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm,
                         cudaStream_t stream);
HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                             HcclReduceOp op, HcclComm comm, cudaStream_t stream);
HcclResult HcclReduceScatterV(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf,
                              uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                              cudaStream_t stream);
HcclResult HcclScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root,
                       HcclComm comm, cudaStream_t stream);
HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm,
                         cudaStream_t stream);
HcclResult HcclAllGatherV(void *sendBuf, uint64_t sendCount, void *recvBuf, const void *recvCounts,
                          const void *recvDispls, HcclDataType dataType, HcclComm comm, cudaStream_t stream);
HcclResult HcclSend(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm,
                    cudaStream_t stream);
HcclResult HcclRecv(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm,
                    cudaStream_t stream);
HcclResult HcclAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType,
                          const void *recvBuf, HcclDataType recvType, HcclComm comm, cudaStream_t stream);
HcclResult HcclAlltoAllV(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType,
                         const void *recvBuf, const void *recvCounts, const void *rdispls, HcclDataType recvType,
                         HcclComm comm, cudaStream_t stream);
HcclResult HcclAlltoAll(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf,
                        uint64_t recvCount, HcclDataType recvType, HcclComm comm, cudaStream_t stream);
HcclResult HcclReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                      uint32_t root, HcclComm comm, cudaStream_t stream);
HcclResult HcclBatchSendRecv(HcclSendRecvItem *sendRecvInfo, uint32_t itemNum, HcclComm comm, cudaStream_t stream);
HcclResult HcclBarrier(HcclComm comm, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
