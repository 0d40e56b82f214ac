#include "launch.h"
#include "../exec/copy_engine.h"
namespace hccl {
const std::vector<SmAlgoDesc> &SmAlgorithms() { static std::vector<SmAlgoDesc> v; return v; }
HcclResult SmOrchestrate(Comm *, OpParam &, const std::string &) { return HCCL_E_UNAVAIL; }
uint32_t SmDefaultCtas(HcclCMDType, const std::string &, uint64_t, uint32_t) { return 0; }
HcclResult CopyEngineRun(Comm *, const Plan &, const ExecBuffers &, cudaStream_t) { return HCCL_E_UNAVAIL; }
}
