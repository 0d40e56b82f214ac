// Operator dispatch core: readiness gate, single-rank shortcut, selector, consistency check, executor lookup,
// engine fallback with a sticky cache, DFX registration (reference: src/ops/op_common/op_common.cc:78-126 Selector,
// :557-688 HcclExecOp, :497-512,563-575 fallback + sticky cache, :2148-2201 SingleRankProc, :2244-2279 algTag).
#pragma once
#include "../core/comm.h"
#include "op_param.h"

namespace hccl {

HcclResult HcclExecOp(Comm *c, OpParam &p);
HcclResult SingleRankProc(Comm *c, OpParam &p);
HcclResult SelectAlgorithm(Comm *c, OpParam &p, const std::vector<HcclCommEngine> &excluded);
// Cross-rank parameter consistency (reference: src/common/inconsistent_check.cc:72-168).
HcclResult CheckOpConsistency(Comm *c, const OpParam &p);
HcclResult CompareOpExchangeInfos(const std::vector<OpExchangeInfo> &all, uint32_t myRank, std::string *why);
void FillOpExchangeInfo(Comm *c, const OpParam &p, OpExchangeInfo *info);
bool StreamIsCapturing(cudaStream_t s);
// Invalidates every cached launch list (tuning table or algorithm configuration changed).
void BumpSelectionGeneration();
HcclResult LocalCopyAsync(Comm *c, void *dst, const void *src, uint64_t bytes, cudaStream_t s);
// Operator retry (op_retry.cc): keeps a copy of the call for CommOpRetry.
void RecordOpForRetry(Comm *c, const OpParam &p);

}  // namespace hccl
