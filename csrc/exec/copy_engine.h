// Copy-engine executor: runs schedule IR on a CUDA communicator with host-issued work only -- peer copies through
// the DMA engines (cudaMemcpyAsync between peer-mapped heaps), small reduce kernels, and one-thread flag kernels
// with bounded waits for POST / WAIT. The B200 stand-in for HCCL's AICPU + SDMA path, useful when SMs must stay
// free for compute and as the fallback engine of the selector cascade.
#pragma once
#include "../core/comm.h"
#include "host_engine.h"
#include "plan.h"

namespace hccl {
HcclResult CopyEngineRun(Comm *c, const Plan &plan, const ExecBuffers &bufs, cudaStream_t stream);
}
