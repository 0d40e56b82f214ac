// Argument block of the collective kernels and the host-side launch description.
// One SmLaunch = one kernel launch = one chunk of an operator; SmPlanOp() turns an operator call into the list of
// launches (pure host arithmetic, identical on every rank, unit-testable without a GPU).
#pragma once
#include <stdint.h>
#include <functional>
#include <string>
#include <vector>
#include "../core/dev_comm.h"
#include "../exec/op_param.h"

namespace hccl {

enum SmKernelId : uint32_t {
    K_ALLREDUCE_ONESHOT = 0,
    K_ALLREDUCE_TWOSHOT,
    K_ALLREDUCE_NVLS_ONESHOT,
    K_ALLREDUCE_NVLS_TWOSHOT,
    K_ALLGATHER_V,            // also AllGather
    K_REDUCESCATTER_V,        // also ReduceScatter
    K_REDUCESCATTER_NVLS,
    K_BROADCAST,
    K_BROADCAST_NVLS,
    K_REDUCE,
    K_SCATTER,
    K_ALLTOALL_V,             // also AlltoAll / AlltoAllVC
    K_BARRIER,
    K_SEND,
    K_RECV,
    K_BATCH_SEND_RECV,
    K_ALLREDUCE_PIPE,         // warp-specialised pipelines (pipelined.cuh): any payload in one launch
    K_ALLREDUCE_PIPE_NVLS,
    K_REDUCESCATTER_PIPE,     // also ReduceScatterV
    K_REDUCESCATTER_PIPE_NVLS,
    K_ALLGATHER_PIPE,         // also AllGatherV
    K_ALLGATHER_PIPE_NVLS,
    K_ALLTOALL_PIPE,          // AlltoAll with uniform counts
    K_ALLREDUCE_RING,         // reduce-scatter + all-gather around the ring (comparator for the mesh kernels)
    K_ALLREDUCE_CONCURRENT,   // two-shot on two sub-grids: both parts by peer stores (no multicast mapping)
    K_ALLREDUCE_CONCURRENT_NVLS,   // ... the first part switch-reduced, the second by peer stores
    // zero-copy forms: the user buffers are registered windows of the symmetric heap (same offset on every rank), so peers and
    // the switch read / write them directly and nothing is staged through the CCL scratch
    K_ALLREDUCE_ZC, K_ALLREDUCE_ZC_NVLS,
    K_REDUCESCATTER_ZC, K_REDUCESCATTER_ZC_NVLS,
    K_ALLGATHER_ZC, K_ALLGATHER_ZC_NVLS,
    K_BROADCAST_ZC, K_BROADCAST_ZC_NVLS,
    K_COUNT
};

constexpr int kP2pBlocks = kP2pCtas;  // CTAs per point-to-point transfer; each owns 1/8 of a mailbox slot
constexpr int kMaxBatchItems = 24;
constexpr uint64_t kA2aMetaBytes = 4 << 10;     // tail of the CCL half reserved for the AlltoAllV round counts (one word per channel)

struct CollArgs {
    const void *in;
    void *out;
    uint64_t count;           // elements in this chunk
    uint64_t bytes;           // count * elemSize
    uint32_t elemSize;
    uint32_t root;
    uint32_t op;              // HcclReduceOp
    uint32_t peer;            // Send / Recv
    uint64_t pipeSub;         // pipelined kernels: bytes of one sub-chunk per (slice, channel), a multiple of 128
    // per-rank byte counts / offsets (V-form kernels; the plain forms fill them uniformly)
    uint64_t sendBytes[kMaxRanks];
    uint64_t sendOff[kMaxRanks];
    uint64_t recvBytes[kMaxRanks];
    uint64_t recvOff[kMaxRanks];
    // concurrent kernels: the first splitBytes of the payload go to the first splitCtas CTAs (first algorithm)
    uint64_t splitBytes;
    uint32_t splitCtas;
    uint32_t pad1;
    // zero-copy kernels: heap offsets of the registered input / output windows (identical on every rank)
    uint64_t inOff, outOff;
    // AlltoAll(V): bytes of the scratch slot each (source, destination) pair owns (identical on every rank, a multiple of 128)
    uint64_t slotBytes;
};

struct BatchItem {
    void *buf;
    uint64_t bytes;
    uint32_t peer;
    uint32_t isSend;          // 1 send, 0 recv, 2 local copy (buf -> buf2)
    void *buf2;
    uint32_t order;           // position among the items of the same (peer, direction) queue
    uint32_t queue;           // queue id; CTAs [queue*kP2pBlocks, (queue+1)*kP2pBlocks) serve it
};
struct BatchArgs {
    uint32_t nItems;
    uint32_t nQueues;
    BatchItem items[kMaxBatchItems];
};

struct SmLaunch {
    SmKernelId kernel;
    HcclDataType dtype;
    uint32_t ctas;
    CollArgs args;
    BatchArgs batch;          // K_BATCH_SEND_RECV only
};

struct SmPlanCtx {
    uint32_t rank, nranks;
    uint64_t cclBytes;
    uint64_t mailboxBytes;
    uint32_t maxCtas;         // 0 = default heuristic
    bool nvls;
    uint32_t splitRatio[2] = {0, 0};   // concurrent algorithms: shares of the first / second part (0:0 = built-in default)
    // zero-copy algorithms: heap offset of a registered window that holds [ptr, ptr + bytes), or false
    std::function<bool(const void *ptr, uint64_t bytes, uint64_t *off)> registeredOffset;
};

// Builds the launch list of one operator for one rank. Returns HCCL_E_NOT_SUPPORT when the algorithm cannot take
// the call (e.g. an NVLS kernel with a payload that is not a multiple of 16 bytes), which makes the dispatch core
// fall back to the next engine -- decided from values every rank shares, so all ranks fall back together.
HcclResult SmPlanOp(const SmPlanCtx &ctx, const OpParam &p, const std::string &algName, std::vector<SmLaunch> *out);
uint32_t SmCtasFor(uint64_t bytes, uint32_t maxCtas);

}  // namespace hccl
