// OpParam: the normalised description of one operator call that travels from the op entry through the
// selector into the executor (reference: src/ops/op_common/inc/alg_param.h:527-609; the trailing varData of
// the reference becomes std::vector members because nothing is shipped to a device CPU here).
#pragma once
#include <cstdint>
#include <string>
#include <vector>
#include "hccl/hccl_comm.h"
#include "hccl/hccl_types.h"

namespace hccl {

enum class OpMode : uint8_t { OPBASE = 0, OFFLOAD = 1 };   // single-op mode / graph (capture) mode

struct OpParam {
    HcclCMDType opType = HCCL_CMD_INVALID;
    std::string tag;                     // "<Op>_<commName>"
    const void *inputPtr = nullptr;
    void *outputPtr = nullptr;
    uint64_t count = 0;                  // elements; meaning per op: AR/Reduce/Bcast count, AG sendCount,
                                         // RS/Scatter recvCount, AlltoAll sendCount per peer
    uint64_t blockStride = 0;            // elements between the per-rank blocks of the gather / scatter forms; 0 = count (a chunk of a
                                         // larger call keeps the stride of the whole call)
    HcclDataType dtype = HCCL_DATA_TYPE_FP32;
    HcclDataType outDtype = HCCL_DATA_TYPE_FP32;
    HcclReduceOp reduceOp = HCCL_REDUCE_SUM;
    uint32_t root = 0;
    uint32_t peer = 0;                   // Send / Recv
    std::vector<uint64_t> sendCounts, sendDispls, recvCounts, recvDispls;   // V variants (elements)
    std::vector<HcclSendRecvItem> items; // BatchSendRecv
    cudaStream_t stream = nullptr;
    OpMode mode = OpMode::OPBASE;
    bool isMc2 = false;
    // graph mode: caller-provided helper streams and scratch
    std::vector<cudaStream_t> slaveStreams;
    void *graphScratch = nullptr;
    uint64_t graphScratchBytes = 0;
    // filled by the selector
    HcclCommEngine engine = HCCL_ENGINE_DEFAULT;
    std::string algName;
    std::string algTag;                  // "<tag>_<alg>_<engine>"
    uint32_t execTimeoutSec = 0;
    uint64_t DataBytes() const;          // payload size used by the selector thresholds
};

}  // namespace hccl
