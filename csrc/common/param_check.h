// Argument validation shared by all op entries.
// Rules reproduced from HCCL (reference: src/common/param_check.cc, src/ops/op_common/op_common.cc:2038-2050 for
// the reduce dtype whitelist, :2091-2107 for the PROD whitelist, src/common/hccl_common.h:42 for SYS_MAX_COUNT,
// src/ops/all_reduce/all_reduce_op.cc:124-149 for null / rank-range checks and the EI0003 error code).
#pragma once
#include <cstdint>
#include "hccl/hccl_types.h"

namespace hccl {
constexpr uint64_t SYS_MAX_COUNT = 0x7FFFFFFFFull;
constexpr uint32_t TAG_MAX_LEN = 255;
constexpr uint32_t ALG_CONFIG_MAX_LEN = 128;

HcclResult HcomCheckCount(uint64_t count);
HcclResult HcomCheckDataType(HcclDataType dataType);                 // any transferable type
HcclResult HcomCheckReduceDataType(HcclDataType dataType, HcclReduceOp op);  // reduce whitelist (+PROD subset)
HcclResult HcomCheckReductionOp(HcclReduceOp op);
HcclResult HcomCheckUserRank(uint32_t totalRanks, uint32_t userRank);
HcclResult HcomCheckTag(const char *tag);
HcclResult HcomCheckOpParam(const char *tag, uint64_t count, HcclDataType dataType);
bool IsReduceDataTypeSupported(HcclDataType dataType);
bool IsProdDataTypeSupported(HcclDataType dataType);
}  // namespace hccl
