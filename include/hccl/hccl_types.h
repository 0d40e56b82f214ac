/*
 * hccl_types.h -- public value types of the B200-native HCCL-compatible collective library.
 *
 * The enumerator names and numeric values follow the public HCCL ABI so that code written
 * against HCCL (reference: include/hccl.h, src/common/hccl_common.h:49-68 for the dtype / reduce-op
 * vocabulary) recompiles unchanged; `aclrtStream` becomes `cudaStream_t`.
 */
#ifndef HCCL_B200_TYPES_H_
#define HCCL_B200_TYPES_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Result codes. 0 is success; every API returns one of these. */
typedef enum {
    HCCL_SUCCESS = 0,
    HCCL_E_PARA = 1,            /* invalid parameter value */
    HCCL_E_PTR = 2,             /* null / invalid pointer */
    HCCL_E_MEMORY = 3,          /* allocation or mapping failure */
    HCCL_E_INTERNAL = 4,        /* library invariant broken */
    HCCL_E_NOT_SUPPORT = 5,     /* dtype / op / algorithm combination not supported */
    HCCL_E_NOT_FOUND = 6,       /* registry or key lookup miss */
    HCCL_E_UNAVAIL = 7,         /* resource (engine, NVLS, peer access) not available */
    HCCL_E_SYSCALL = 8,
    HCCL_E_TIMEOUT = 9,         /* a bounded wait ran out (device flag, bootstrap socket) */
    HCCL_E_OPEN_FILE_FAILURE = 10,
    HCCL_E_TCP_CONNECT = 11,
    HCCL_E_ROCE_CONNECT = 12,
    HCCL_E_TCP_TRANSFER = 13,
    HCCL_E_ROCE_TRANSFER = 14,
    HCCL_E_RUNTIME = 15,        /* CUDA runtime / driver call failed */
    HCCL_E_DRV = 16,
    HCCL_E_PROFILING = 17,
    HCCL_E_CCE = 18,
    HCCL_E_NETWORK = 19,
    HCCL_E_AGAIN = 20,
    HCCL_E_REMOTE = 21,         /* a peer reported an error */
    HCCL_E_SUSPENDING = 22,     /* communicator is suspended; resume it before launching */
    HCCL_E_OPRETRY_FAIL = 23,
    HCCL_E_OOM = 24,
    HCCL_E_RESERVED = 255
} HcclResult;

typedef enum {
    HCCL_REDUCE_SUM = 0,
    HCCL_REDUCE_PROD = 1,
    HCCL_REDUCE_MAX = 2,
    HCCL_REDUCE_MIN = 3,
    HCCL_REDUCE_RESERVED = 255
} HcclReduceOp;

typedef enum {
    HCCL_DATA_TYPE_INT8 = 0,
    HCCL_DATA_TYPE_INT16 = 1,
    HCCL_DATA_TYPE_INT32 = 2,
    HCCL_DATA_TYPE_FP16 = 3,
    HCCL_DATA_TYPE_FP32 = 4,
    HCCL_DATA_TYPE_INT64 = 5,
    HCCL_DATA_TYPE_UINT64 = 6,
    HCCL_DATA_TYPE_UINT8 = 7,
    HCCL_DATA_TYPE_UINT16 = 8,
    HCCL_DATA_TYPE_UINT32 = 9,
    HCCL_DATA_TYPE_FP64 = 10,
    HCCL_DATA_TYPE_BFP16 = 11,
    HCCL_DATA_TYPE_INT128 = 12,
    HCCL_DATA_TYPE_HIF8 = 14,
    HCCL_DATA_TYPE_FP8E4M3 = 15,
    HCCL_DATA_TYPE_FP8E5M2 = 16,
    HCCL_DATA_TYPE_FP8E8M0 = 17,
    HCCL_DATA_TYPE_RESERVED = 255
} HcclDataType;

/* Collective kinds; used by the MC2 resource-context API, the graph-mode API, the selector
 * registry and the DFX op registry. */
typedef enum {
    HCCL_CMD_INVALID = 0,
    HCCL_CMD_BROADCAST = 1,
    HCCL_CMD_ALLREDUCE = 2,
    HCCL_CMD_REDUCE = 3,
    HCCL_CMD_SEND = 4,
    HCCL_CMD_RECEIVE = 5,
    HCCL_CMD_ALLGATHER = 6,
    HCCL_CMD_REDUCE_SCATTER = 7,
    HCCL_CMD_ALLTOALLV = 8,
    HCCL_CMD_ALLTOALLVC = 9,
    HCCL_CMD_ALLTOALL = 10,
    HCCL_CMD_GATHER = 11,
    HCCL_CMD_SCATTER = 12,
    HCCL_CMD_BATCH_SEND_RECV = 13,
    HCCL_CMD_BARRIER = 14,
    HCCL_CMD_ALLGATHER_V = 15,
    HCCL_CMD_REDUCE_SCATTER_V = 16,
    /* fused compute + collective ops (MC2) and MoE routing */
    HCCL_CMD_ALLGATHER_MATMUL = 32,
    HCCL_CMD_MATMUL_REDUCE_SCATTER = 33,
    HCCL_CMD_MATMUL_ALLREDUCE = 34,
    HCCL_CMD_MOE_DISPATCH = 35,
    HCCL_CMD_MOE_COMBINE = 36,
    HCCL_CMD_MAX = 37
} HcclCMDType;

/* Which machinery executes an op ("expansion mode" in HCCL terms).
 *   SM          hand-written sm_100a kernels doing peer loads/stores from inside the kernel
 *   NVLS        the same kernels using multimem.* through the NVSwitch multicast object
 *   COPY_ENGINE host-issued schedule (task list) of peer copies + small reduce kernels
 *   HOST        CPU simulation backend (ranks are threads/processes, heap is shared memory)
 */
typedef enum {
    HCCL_ENGINE_DEFAULT = 0,
    HCCL_ENGINE_HOST = 1,
    HCCL_ENGINE_COPY_ENGINE = 2,
    HCCL_ENGINE_SM = 3,
    HCCL_ENGINE_NVLS = 4,
    HCCL_ENGINE_RESERVED = 255
} HcclCommEngine;

typedef enum { HCCL_SEND = 0, HCCL_RECV = 1, HCCL_SEND_RECV_RESERVED } HcclSendRecvType;

typedef struct HcclSendRecvItemDef {
    HcclSendRecvType sendRecvType;
    void *buf;
    uint64_t count;
    HcclDataType dataType;
    uint32_t remoteRank;
} HcclSendRecvItem;

#define HCCL_ROOT_INFO_BYTES 4108
typedef struct HcclRootInfoDef {
    char internal[HCCL_ROOT_INFO_BYTES];
} HcclRootInfo;

typedef void *HcclComm;

#define HCCL_COMM_NAME_MAX 128
#define HCCL_COMM_CONFIG_MAGIC 0xf0f0f0f0u

/* Per-communicator configuration; overrides the environment when a field is set.
 * Fill with HcclCommConfigInit() first. */
typedef struct HcclCommConfigDef {
    uint32_t size;                 /* sizeof(HcclCommConfig), for ABI checks */
    uint32_t magic;
    uint32_t version;
    uint32_t hcclBufferSize;       /* MB per CCL scratch buffer (two per comm); 0 = env/default (200) */
    uint32_t hcclDeterministic;    /* 0 off, 1 on (fixed order), 2 strict; 0xffffffff = env */
    char hcclCommName[HCCL_COMM_NAME_MAX];
    char hcclUdi[HCCL_COMM_NAME_MAX];
    uint32_t hcclOpExpansionMode;  /* HcclCommEngine; 0 = env/default */
    uint32_t hcclRdmaTrafficClass; /* accepted, unused on a single NVSwitch box */
    uint32_t hcclRdmaServiceLevel; /* accepted, unused */
    uint32_t hcclWorldRankID;
    uint64_t hcclJobID;
    uint32_t hcclExecTimeoutSec;   /* 0 = env/default */
    uint32_t hcclBackend;          /* 0 auto (CUDA when a device is current, else host sim), 1 sim, 2 cuda */
    uint32_t reserved[16];
} HcclCommConfig;

#define HCCL_CONFIG_NOT_SET 0xffffffffu

#ifdef __cplusplus
}
#endif
#endif /* HCCL_B200_TYPES_H_ */
