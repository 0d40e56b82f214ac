#include "copy_engine.h"
namespace hccl { HcclResult CopyEngineRun(Comm *, const Plan &, const ExecBuffers &, cudaStream_t) { return HCCL_E_UNAVAIL; } }
