// Copy-engine executor: runs schedule IR on a CUDA communicator with host-issued work only -- peer copies through
// the DMA engines (cudaMemcpyAsync between peer-mapped heaps), small reduce kernels, and one-thread flag kernels
// with bounded waits for POST / WAIT. The B200 stand-in for HCCL's AICPU + SDMA path, useful when SMs must stay
// free for compute and as the fallback engine of the selector cascade.
#pragma once
#include "../core/comm.h"
#include "host_engine.h"
#include "plan.h"

namespace hccl {
// isCollective: every rank of the communicator runs a plan of this operator (the plan is then bracketed by an all-rank notify
// barrier); false for point-to-point schedules, which this engine refuses (their queues would be launches that wait on one
// another on one GPU).
HcclResult CopyEngineRun(Comm *c, const Plan &plan, const ExecBuffers &bufs, cudaStream_t stream, bool isCollective);
}
