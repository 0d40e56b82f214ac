/*
 * hccl_comm.h -- communicator management.
 *
 * In HCCL these entry points live in the separate "hcomm" library and are reached from the operator
 * layer through dlopen (reference: src/common/hcomm_dlsym/hcomm_dlsym.cc:62-83; usage in
 * examples/02_collectives/01_allreduce/main.cc:77,122). Here they are part of the same library: a
 * communicator owns a TCP bootstrap ring, a peer-mapped symmetric heap (CUDA VMM allocations exported
 * as POSIX file descriptors, optionally bound to an NVSwitch multicast object), a flag arena with
 * device-resident epochs, and the caches the operator layer keeps per communicator.
 */
#ifndef HCCL_B200_COMM_H_
#define HCCL_B200_COMM_H_

#include "hccl_types.h"

#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st *cudaStream_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Rank 0 creates the rendezvous blob (ip, port, nonce) that is shared out of band. */
HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo);
HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm);
HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank,
                                      const HcclCommConfig *config, HcclComm *comm);
/* Rank-table (JSON file path) based init; the table lists servers and their device ranks. */
HcclResult HcclCommInitClusterInfo(const char *clusterInfo, uint32_t rank, HcclComm *comm);
HcclResult HcclCommInitClusterInfoConfig(const char *clusterInfo, uint32_t rank, const HcclCommConfig *config,
                                         HcclComm *comm);
/* Single-process convenience: one communicator per listed device, one thread each internally. */
HcclResult HcclCommInitAll(uint32_t ndev, int32_t *devices, HcclComm *comms);
HcclResult HcclCreateSubCommConfig(HcclComm *comm, uint32_t rankNum, uint32_t *rankIds, uint64_t subCommId,
                                   uint32_t subCommRankId, HcclCommConfig *config, HcclComm *subComm);
HcclResult HcclCommDestroy(HcclComm comm);
void HcclCommConfigInit(HcclCommConfig *config);

HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize);
HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank);
HcclResult HcclGetCommName(HcclComm comm, char *commName);
/* The per-communicator scratch ("CCL buffer") that every peer can address. */
HcclResult HcclGetHcclBuffer(HcclComm comm, void **addr, uint64_t *size);
const char *HcclGetErrorString(HcclResult code);

/* Communicator state machine: READY -> SUSPENDING (after a device-side timeout or HcclCommSuspend)
 * -> READY again after HcclCommResume (re-zeroes flags and epochs on every rank). */
typedef enum { HCCL_COMM_STATUS_READY = 0, HCCL_COMM_STATUS_SUSPENDING = 1, HCCL_COMM_STATUS_INVALID = 2 } HcclCommStatus;
HcclResult HcclCommGetStatus(HcclComm comm, HcclCommStatus *status);
HcclResult HcclCommSuspend(HcclComm comm);
HcclResult HcclCommResume(HcclComm comm);
/* Reads the device status word after the stream has drained; returns HCCL_E_TIMEOUT (and suspends
 * the communicator) when a kernel gave up waiting. Cheap; never blocks. */
HcclResult HcclGetCommAsyncError(HcclComm comm, HcclResult *asyncError);

/* Zero-copy support: registered buffers live in (or are mapped into) the symmetric address space so
 * peers can read/write them directly. HcclCommSymAlloc returns memory from the symmetric heap. */
HcclResult HcclCommSymAlloc(HcclComm comm, uint64_t bytes, void **ptr);
/* Caps the grid of this communicator's collective kernels (0 = the kernels' own heuristics; the HCCL_MAX_CTAS environment value is the
 * initial setting). A gradient all-reduce that overlaps a backward pass wants few CTAs so that the GEMMs keep their SMs. */
HcclResult HcclCommSetMaxCtas(HcclComm comm, uint32_t maxCtas);
HcclResult HcclCommSymFree(HcclComm comm, void *ptr);
HcclResult HcclSymWinGetPeerPointer(HcclComm comm, void *localPtr, uint32_t peer, void **peerPtr);
HcclResult HcclSymGetMulticastPointer(HcclComm comm, void *localPtr, void **mcPtr);

/* Host simulation backend only: wait for the communicator's worker queue to drain. With CUDA use
 * cudaStreamSynchronize on the stream given to the op. */
HcclResult HcclSimStreamSynchronize(HcclComm comm);

#ifdef __cplusplus
}
#endif
#endif
