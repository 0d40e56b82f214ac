// Host-side interface of the SM / NVLS engine: one fused kernel launch per chunk, issued on the caller's stream.
// This is the B200 counterpart of HCCL's vector-core engine launch (reference: src/ops/op_common/op_common.cc:888-911
// HcclAivKernelEntranceLaunch; src/ops/op_common/template/aiv/hccl_aiv_utils.cc:931-953 ExecuteKernelLaunch):
// kernels take the device-resident DevComm (peer heap table, flags, epochs) plus a small by-value argument block.
#pragma once
#include <string>
#include <vector>
#include "../core/comm.h"
#include "../exec/op_param.h"

namespace hccl {

struct SmAlgoDesc {
    const char *name;
    HcclCMDType op;
    bool nvls;
};
const std::vector<SmAlgoDesc> &SmAlgorithms();

// Runs the whole operator (chunk loop inside) with the named SM / NVLS algorithm.
HcclResult SmOrchestrate(Comm *c, OpParam &p, const std::string &algName);
// Issues one planned launch on `stream` (used by the dispatch core to replay a cached launch list).
struct SmLaunch;
struct DevComm;
HcclResult SmIssueLaunch(const DevComm *devComm, const SmLaunch &l, cudaStream_t stream);
// While non-null on the calling thread, SmOrchestrate copies the launch list it issued here.
extern thread_local std::vector<SmLaunch> *g_captureLaunches;
// Grid size the engine would use (selector hint / graph-mode resource query).
uint32_t SmDefaultCtas(HcclCMDType op, const std::string &algName, uint64_t bytes, uint32_t nranks);

}  // namespace hccl
