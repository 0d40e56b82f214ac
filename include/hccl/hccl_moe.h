/*
 * hccl_moe.h -- expert-parallel MoE token dispatch / combine as fused kernels.
 *
 * HCCL offers AlltoAllV with host-resident count arrays for this job (reference: include/hccl.h:180-223; the vector-core
 * kernel src/ops/all_to_all_v/template/aiv/kernel/aiv_all_to_all_v_mesh_1D.h:16-271). Routing decisions live on the device,
 * so here each direction is ONE kernel that does everything on the device:
 *   dispatch  histogram of the routing table -> count exchange through the symmetric heap -> every (token, k) row is written
 *             straight into its slot of the destination rank's receive buffer, grouped by expert, ordered by source rank
 *             and token (deterministic layout), optionally quantised to MXFP8 (e4m3 payload, 1x32 blocks, e8m0 scales)
 *   combine   every rank pulls the expert outputs of its own tokens from the peers and forms the top-k weighted sum in
 *             fp32 (fixed k order), writing bf16.
 * Receive and expert-output buffers live in the communicator's symmetric heap and are handed out as device pointers
 * (no copy on either side of the expert computation).
 */
#ifndef HCCL_B200_MOE_H_
#define HCCL_B200_MOE_H_

#include "hccl_comm.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct HcclMoeConfigDef {
    uint32_t numExperts;       /* global; a multiple of the rank count; at most 320 */
    uint32_t topK;             /* at most 16 */
    uint32_t hidden;           /* a multiple of 256 */
    uint32_t maxTokens;        /* tokens per rank per call, upper bound */
    uint32_t maxRecvRows;      /* capacity of the receive buffer in rows; 0 = 2 * maxTokens * topK */
    uint32_t mxfp8;            /* 1: dispatch payload is e4m3 with e8m0 scales per 32 values */
    uint32_t reserved[4];
} HcclMoeConfig;

typedef void *HcclMoeHandle;

/* Collective: allocates the symmetric buffers. */
HcclResult HcclMoeCreate(HcclComm comm, const HcclMoeConfig *config, HcclMoeHandle *handle);
HcclResult HcclMoeDestroy(HcclMoeHandle handle);

/* x: [numTokens, hidden] bf16; topkIdx: [numTokens, topK] int32 expert ids. Device pointers returned:
 *   recvX       [rows, hidden] bf16 (or e4m3) grouped by local expert
 *   recvScales  [rows, hidden/32] e8m0 (mxfp8 only, else NULL)
 *   recvCounts  [numExperts / ranks] int32 rows per local expert
 *   recvSrc     [rows] int32 = (source rank << 24) | source token */
HcclResult HcclMoeDispatch(HcclMoeHandle handle, const void *x, const int32_t *topkIdx, uint32_t numTokens, void **recvX, void **recvScales,
                           int32_t **recvCounts, int32_t **recvSrc, cudaStream_t stream);
/* Symmetric buffer [maxRecvRows, hidden] bf16 the caller fills with expert outputs, row i answering recvX row i. */
HcclResult HcclMoeGetExpertOutBuffer(HcclMoeHandle handle, void **y);
/* out[t] = sum_k topkWeights[t, k] * y(row the dispatch gave (t, k)); topkWeights [numTokens, topK] fp32; out bf16. */
HcclResult HcclMoeCombine(HcclMoeHandle handle, const float *topkWeights, void *out, uint32_t numTokens, cudaStream_t stream);

/* Single-GPU emulation (tests): all ranks in one cooperative launch. xs / idxs / weights / outs are per-rank pointers;
 * `identityExperts` copies recvX to the expert-output buffer between dispatch and combine. */
HcclResult HcclEmuMoeRoundTrip(void *emu, const HcclMoeConfig *config, void **xs, void **idxs, void **weights, void **outs, uint32_t numTokens,
                               void **recvCountsOut, uint32_t ctasPerRank);

#ifdef __cplusplus
}
#endif
#endif
