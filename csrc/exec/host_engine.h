// Host engine: interprets schedule IR on the CPU over the shared-memory symmetric heap (simulation backend).
// Plays the role HCCL's AICPU executor plays on the device CPU (reference: src/ops/op_common/template/aicpu/
// kernel_launch.cc:242-549 runs Orchestrate and issues the primitives), with real data movement so numerics
// can be checked against an fp64 oracle without a GPU. Reductions that the reference does on the CPU for
// int64/uint64/fp64/PROD (alg_data_trans_wrapper.h:79-89) are all done here.
#pragma once
#include "../core/comm.h"
#include "plan.h"

namespace hccl {

struct ExecBuffers {
    char *in = nullptr;
    char *out = nullptr;
    uint32_t cclHalf = 0;
};

HcclResult HostEngineRun(Comm *c, const Plan &plan, const ExecBuffers &bufs);
// dst = dst (op) src over `bytes` of `dtype`; the single reduce routine of the host path and the test oracles.
HcclResult HostReduce(void *dst, const void *src, uint64_t bytes, HcclDataType dtype, HcclReduceOp op);

}  // namespace hccl
