/*
 * hccl_noalloc.h -- an all-reduce across buffers of ONE GPU that never allocates memory.
 *
 * This entry point has no counterpart in HCCL; it exists for callers of this library that must not (or cannot) call
 * cudaMalloc: serving processes that have handed the whole device to their own pool allocator, so that a driver
 * allocation would fail or fragment the pool, and latency-critical loops that cannot afford the device-wide
 * synchronisation cudaMalloc / cudaFree imply.
 *
 * It runs the same two-shot all-reduce kernel the communicator uses (reduce-scatter by stores into per-rank slots,
 * rank-ordered reduction, all-gather by loads) with every "rank" being one (send, recv) buffer pair on the current
 * device. The scratch that kernel needs -- control blocks, flag words and the staging halves, normally part of a
 * communicator's heap -- lives in a fixed array inside the library image (about 5 MiB, held by every GPU that loads the
 * library until the process exits).
 *
 * Limits and rules:
 *   - 2 to 4 buffer pairs, at most HCCL_NOALLOC_MAX_BYTES (256 KiB) per buffer; larger requests are rejected with
 *     HCCL_E_PARA and a log line, nothing is launched.
 *   - Reducible data types and operations as for HcclAllReduce.
 *   - The first call on a device looks up the device address of the scratch array; make that first call before any
 *     stream capture begins on that device.
 *   - All calls share the one scratch array. Each call clears the part it needs at its start (on the given stream), so
 *     calls issued on one stream are independent, but calls whose kernels could overlap on the GPU (different
 *     streams, different host threads) race on the scratch and must be serialised by the caller.
 *   - Asynchronous: returns after enqueueing on `stream`. Neither this function nor anything it calls allocates
 *     device or pinned host memory. The per-call tables travel to the device by value, as parameters of a small set-up
 *     kernel, so no host memory of the caller has to outlive the call.
 *   - The kernel's waits are bounded (2 s). A wait that runs out cannot be reported by the call that launched it, which
 *     has long returned: it leaves a record in the scratch array. HcclLocalAllReduceNoAllocStatus copies those records
 *     to host memory you supply (one 32-byte record per buffer pair, first word 0 = fine, 1 = a wait ran out); it does
 *     not allocate either. Host threads may call both functions concurrently as far as the address look-up goes; the
 *     rule about overlapping kernels above still applies.
 */
#ifndef HCCL_B200_NOALLOC_H_
#define HCCL_B200_NOALLOC_H_

#include "hccl_comm.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_NOALLOC_MAX_BUFFERS 4
#define HCCL_NOALLOC_MAX_BYTES (256u << 10)

/* recvBufs[i] = reduce over j of sendBufs[j], for every i < nBufs (sendBufs[i] == recvBufs[i] is allowed). */
HcclResult HcclLocalAllReduceNoAlloc(const void *const *sendBufs, void *const *recvBufs, uint32_t nBufs, uint64_t count,
                                     HcclDataType dataType, HcclReduceOp op, cudaStream_t stream);


/* Copies nRecords (1..HCCL_NOALLOC_MAX_BUFFERS) 32-byte status records {code, rank, peer, channel, phase, opSeq, observed,
 * expected} of the most recent call into hostRecords, asynchronously on `stream` (synchronise it before reading). */
HcclResult HcclLocalAllReduceNoAllocStatus(void *hostRecords, uint32_t nRecords, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
