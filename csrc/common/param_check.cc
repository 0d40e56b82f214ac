#include <cstdlib>
#include "param_check.h"
#include <cstring>
#include "dtype.h"
#include "log.h"

namespace hccl {

HcclResult HcomCheckCount(uint64_t count)
{
    if (count > SYS_MAX_COUNT) {
        HCCL_ERROR("[EI0003] count %llu exceeds the supported maximum %llu", (unsigned long long)count,
                   (unsigned long long)SYS_MAX_COUNT);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult HcomCheckDataType(HcclDataType t)
{
    if (DataTypeSize(t) == 0) {
        HCCL_ERROR("[EI0003] data type %d is not supported", (int)t);
        return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

// HCCL_STRICT_DTYPE_RULES=1 reproduces the reference's operand rules exactly (no unsigned 8/16/32-bit reductions, PROD
// only for int8/int32/int64/uint64/fp16/fp32/fp64; reference: src/ops/op_common/op_common.cc:2038-2050,2091-2107). By
// default this library accepts the superset its kernels implement.
static bool StrictRules()
{
    static const bool v = [] { const char *e = getenv("HCCL_STRICT_DTYPE_RULES"); return e && *e && *e != '0'; }();
    return v;
}

bool IsReduceDataTypeSupported(HcclDataType t)
{
    if (StrictRules() && (t == HCCL_DATA_TYPE_UINT8 || t == HCCL_DATA_TYPE_UINT16 || t == HCCL_DATA_TYPE_UINT32)) return false;
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_INT64:
        case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_FP32: case HCCL_DATA_TYPE_FP64:
        case HCCL_DATA_TYPE_BFP16: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_UINT32: return true;
        default: return false;
    }
}

bool IsProdDataTypeSupported(HcclDataType t)
{
    // every reducible type multiplies here (the reference excludes int16 and bf16: an engine limit this hardware lacks)
    if (StrictRules() && (t == HCCL_DATA_TYPE_INT16 || t == HCCL_DATA_TYPE_BFP16)) return false;
    return IsReduceDataTypeSupported(t);
}

HcclResult HcomCheckReductionOp(HcclReduceOp op)
{
    if (op != HCCL_REDUCE_SUM && op != HCCL_REDUCE_PROD && op != HCCL_REDUCE_MAX && op != HCCL_REDUCE_MIN) {
        HCCL_ERROR("[EI0003] reduce op %d is not supported", (int)op);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult HcomCheckReduceDataType(HcclDataType t, HcclReduceOp op)
{
    CHK_RET(HcomCheckReductionOp(op));
    if (!IsReduceDataTypeSupported(t)) {
        HCCL_ERROR("[EI0003] data type %s cannot be reduced", DataTypeName(t));
        return HCCL_E_NOT_SUPPORT;
    }
    if (op == HCCL_REDUCE_PROD && !IsProdDataTypeSupported(t)) {
        HCCL_ERROR("[EI0003] data type %s does not support prod", DataTypeName(t));
        return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

HcclResult HcomCheckUserRank(uint32_t totalRanks, uint32_t userRank)
{
    if (userRank >= totalRanks) {
        HCCL_ERROR("[EI0003] rank %u is outside [0, %u)", userRank, totalRanks);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult HcomCheckTag(const char *tag)
{
    CHK_PTR_NULL(tag);
    size_t n = strnlen(tag, TAG_MAX_LEN + 1);
    if (n == 0 || n > TAG_MAX_LEN) {
        HCCL_ERROR("[EI0003] tag length %zu is outside [1, %u]", n, TAG_MAX_LEN);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult HcomCheckOpParam(const char *tag, uint64_t count, HcclDataType dataType)
{
    CHK_RET(HcomCheckTag(tag));
    CHK_RET(HcomCheckCount(count));
    return HcomCheckDataType(dataType);
}

}  // namespace hccl
