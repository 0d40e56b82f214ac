// Data-type / reduce-op tables and scalar conversion helpers shared by the host engines.
// The size table and string names follow HCCL's (reference: src/ops/op_common/inc/alg_param.h:43-45,
// src/common/hccl_common.h:49-68).
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include "hccl/hccl_types.h"

namespace hccl {

inline uint32_t DataTypeSize(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_HIF8:
        case HCCL_DATA_TYPE_FP8E4M3: case HCCL_DATA_TYPE_FP8E5M2: case HCCL_DATA_TYPE_FP8E8M0: return 1;
        case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_FP16:
        case HCCL_DATA_TYPE_BFP16: return 2;
        case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_FP32: return 4;
        case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP64: return 8;
        case HCCL_DATA_TYPE_INT128: return 16;
        default: return 0;
    }
}

inline const char *DataTypeName(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: return "int8";
        case HCCL_DATA_TYPE_INT16: return "int16";
        case HCCL_DATA_TYPE_INT32: return "int32";
        case HCCL_DATA_TYPE_FP16: return "float16";
        case HCCL_DATA_TYPE_FP32: return "float32";
        case HCCL_DATA_TYPE_INT64: return "int64";
        case HCCL_DATA_TYPE_UINT64: return "uint64";
        case HCCL_DATA_TYPE_UINT8: return "uint8";
        case HCCL_DATA_TYPE_UINT16: return "uint16";
        case HCCL_DATA_TYPE_UINT32: return "uint32";
        case HCCL_DATA_TYPE_FP64: return "float64";
        case HCCL_DATA_TYPE_BFP16: return "bfloat16";
        case HCCL_DATA_TYPE_INT128: return "int128";
        case HCCL_DATA_TYPE_HIF8: return "hif8";
        case HCCL_DATA_TYPE_FP8E4M3: return "fp8e4m3";
        case HCCL_DATA_TYPE_FP8E5M2: return "fp8e5m2";
        case HCCL_DATA_TYPE_FP8E8M0: return "fp8e8m0";
        default: return "reserved";
    }
}

inline const char *ReduceOpName(HcclReduceOp op)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return "sum";
        case HCCL_REDUCE_PROD: return "prod";
        case HCCL_REDUCE_MAX: return "max";
        case HCCL_REDUCE_MIN: return "min";
        default: return "reserved";
    }
}

inline const char *CmdName(HcclCMDType c)
{
    switch (c) {
        case HCCL_CMD_BROADCAST: return "Broadcast";
        case HCCL_CMD_ALLREDUCE: return "AllReduce";
        case HCCL_CMD_REDUCE: return "Reduce";
        case HCCL_CMD_SEND: return "Send";
        case HCCL_CMD_RECEIVE: return "Recv";
        case HCCL_CMD_ALLGATHER: return "AllGather";
        case HCCL_CMD_REDUCE_SCATTER: return "ReduceScatter";
        case HCCL_CMD_ALLTOALLV: return "AlltoAllV";
        case HCCL_CMD_ALLTOALLVC: return "AlltoAllVC";
        case HCCL_CMD_ALLTOALL: return "AlltoAll";
        case HCCL_CMD_GATHER: return "Gather";
        case HCCL_CMD_SCATTER: return "Scatter";
        case HCCL_CMD_BATCH_SEND_RECV: return "BatchSendRecv";
        case HCCL_CMD_BARRIER: return "Barrier";
        case HCCL_CMD_ALLGATHER_V: return "AllGatherV";
        case HCCL_CMD_REDUCE_SCATTER_V: return "ReduceScatterV";
        case HCCL_CMD_ALLGATHER_MATMUL: return "AllGatherMatmul";
        case HCCL_CMD_MATMUL_REDUCE_SCATTER: return "MatmulReduceScatter";
        case HCCL_CMD_MATMUL_ALLREDUCE: return "MatmulAllReduce";
        case HCCL_CMD_MOE_DISPATCH: return "MoeDispatch";
        case HCCL_CMD_MOE_COMBINE: return "MoeCombine";
        default: return "Invalid";
    }
}

// fp16 / bf16 <-> fp32 on the host (round-to-nearest-even), used by the host engines and oracles.
inline float Bf16ToFloat(uint16_t v)
{
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t FloatToBf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
inline float Fp16ToFloat(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t FloatToFp16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    int32_t exp = (int32_t)((u >> 23) & 0xffu) - 127 + 15;
    uint32_t man = u & 0x7fffffu;
    if (((u >> 23) & 0xffu) == 0xffu) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
}

}  // namespace hccl
