/*
 * hccl_mc2.h -- matmul + communication ("MC2") interface.
 *
 * Part 1 keeps HCCL's argument / resource-context API (reference: include/hccl_mc2.h:25-82, implementation
 * src/common/hccl_mc2.cc:21-165): an opaque HcclOpArgs blob with setters, and HcclCreateOpResCtx which returns a
 * device-resident context (peer heap table, flag arena, workspace window) that a caller's own fused kernel can use to
 * talk to the other ranks.
 * Part 2 is new: the fused operators themselves, each ONE sm_100a kernel that overlaps tcgen05 GEMM tiles with the
 * peer-memory traffic of the collective (HCCL ships no such kernels; they live in external operator libraries there).
 */
#ifndef HCCL_B200_MC2_H_
#define HCCL_B200_MC2_H_

#include "hccl_comm.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- Part 1: argument blob + resource context ------------------------------------------------------------------ */
HcclResult HcclKfcAllocOpArgs(void **opArgs);
HcclResult HcclKfcFreeOpArgs(void *opArgs);
HcclResult HcclKfcOpArgsSetSrcDataType(void *opArgs, uint8_t srcDataType);
HcclResult HcclKfcOpArgsSetDstDataType(void *opArgs, uint8_t dstDataType);
HcclResult HcclKfcOpArgsSetReduceType(void *opArgs, uint32_t reduceType);
HcclResult HcclKfcOpArgsSetCount(void *opArgs, uint64_t count);
HcclResult HcclKfcOpArgsSetAlgConfig(void *opArgs, char *algConfig);   /* at most 128 characters */
HcclResult HcclKfcOpArgsSetCommEngine(void *opArgs, uint8_t commEngine); /* HCCL_ENGINE_SM or HCCL_ENGINE_NVLS */
HcclResult HcclCreateOpResCtx(HcclComm comm, uint8_t opType, void *opArgs, void **opResCtx);

/* Layout of the device-resident context returned by HcclCreateOpResCtx (read it from device code). */
typedef struct HcclOpResCtxDef {
    uint32_t magic;             /* 'MC2C' */
    uint32_t opType;
    uint32_t rank, nranks;
    uint32_t srcDataType, dstDataType, reduceType, commEngine;
    uint64_t count;
    uint64_t heapBytes;
    void *heap[32];             /* heap[r]: rank r's symmetric heap as mapped on this device */
    void *mcHeap;               /* multicast mapping, or NULL */
    uint64_t workspaceOff;      /* window inside every heap reserved for this context */
    uint64_t workspaceBytes;
    uint64_t flagOff;           /* 64 KB of zero-initialised flag words inside the window */
    uint64_t timeoutNs;         /* bound the library uses for its own waits */
    char algConfig[128];
} HcclOpResCtx;

/* ---- Part 2: fused operators (bf16 here, block-scaled fp8 in part 3; weights are [N, K] row-major, i.e. K contiguous) ---------------------------- */
/* C[M,N] = A[M,K] * B[N,K]^T on one GPU (the building block; also the N = 1 degenerate case of the fused ops). */
HcclResult HcclGemmBf16(const void *a, const void *b, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32, cudaStream_t stream);
/* variant 0 = automatic, 1 = one-CTA 128 x BN tiles, 2 = 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2) */
HcclResult HcclGemmBf16Variant(const void *a, const void *b, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32, int variant, cudaStream_t stream);
HcclResult HcclGemmCheckError(void);
/* Kernels this library has launched in this process so far (all operators; benchmarks report the delta over a region). */
uint64_t HcclGetKernelLaunchCount(void);

/* out[nranks*mLocal, n] = AllGather_rows(aLocal[mLocal, k]) * b[n, k]^T. gathered (optional, [nranks*mLocal, k]) receives the
 * gathered activations for reuse in the backward pass. */
HcclResult HcclAllGatherMatmul(const void *aLocal, const void *b, void *out, void *gathered, uint64_t mLocal, uint64_t n, uint64_t k,
                               HcclDataType dataType, HcclComm comm, cudaStream_t stream);
/* out[m/nranks, n] = ReduceScatter_rows(a[m, kLocal] * b[n, kLocal]^T), sum in rank order. */
HcclResult HcclMatmulReduceScatter(const void *a, const void *b, void *out, uint64_t m, uint64_t n, uint64_t kLocal, HcclDataType dataType,
                                   HcclComm comm, cudaStream_t stream);
/* out[m, n] = AllReduce(a[m, kLocal] * b[n, kLocal]^T), sum in rank order (decode-sized m). */
HcclResult HcclMatmulAllReduce(const void *a, const void *b, void *out, uint64_t m, uint64_t n, uint64_t kLocal, HcclDataType dataType,
                               HcclComm comm, cudaStream_t stream);


/* ---- Part 3: block-scaled fp8 (MXFP8: e4m3 elements, one e8m0 scale per 1 x 32 block of K) ------------------------
 * Operand format of a [rows, k] matrix, k a multiple of 128: `payload` = rows x k bytes row-major; `scales` =
 * HcclMxfp8ScaleBytes(rows, k) bytes in 512-byte atoms [ceil(rows/128)][k/128], the scale of row r, 32-element block kb at
 * atom (r/128, kb/4), byte (r%32)*16 + ((r%128)/32)*4 + kb%4. The tensor cores apply the scales (tcgen05 block_scale). */
uint64_t HcclMxfp8ScaleBytes(uint64_t rows, uint64_t k);
/* bf16 [rows, k] -> payload + scales (power-of-two scale from the block's largest magnitude, saturating e4m3 rounding). */
HcclResult HcclQuantizeMxfp8(const void *in, void *payload, void *scales, uint64_t rows, uint64_t k, cudaStream_t stream);
/* C[m,n] = A[m,k] * B[n,k]^T on one GPU, both operands block-scaled, bf16 (or fp32) result. */
HcclResult HcclGemmMxfp8(const void *a, const void *sfa, const void *b, const void *sfb, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32,
                         cudaStream_t stream);
/* tileN 128 or 256 forces the tile width (0 = automatic). */
HcclResult HcclGemmMxfp8Variant(const void *a, const void *sfa, const void *b, const void *sfb, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32,
                                int tileN, cudaStream_t stream);
/* The three fused operators on block-scaled operands (bf16 results; shapes as for the bf16 forms, k a multiple of 128).
 * AllGatherMatmul moves one byte per element plus the scales between GPUs. */
HcclResult HcclAllGatherMatmulMxfp8(const void *aLocal, const void *sfaLocal, const void *b, const void *sfb, void *out, uint64_t mLocal, uint64_t n,
                                    uint64_t k, HcclComm comm, cudaStream_t stream);
HcclResult HcclMatmulReduceScatterMxfp8(const void *a, const void *sfa, const void *b, const void *sfb, void *out, uint64_t m, uint64_t n, uint64_t kLocal,
                                        HcclComm comm, cudaStream_t stream);
HcclResult HcclMatmulAllReduceMxfp8(const void *a, const void *sfa, const void *b, const void *sfb, void *out, uint64_t m, uint64_t n, uint64_t kLocal,
                                    HcclComm comm, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
