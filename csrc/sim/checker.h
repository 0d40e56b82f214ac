// Offline schedule checker: proves properties of the host-issued schedules without moving data.
//
// Same idea as HCCL's "algorithm analyzer" (reference: test/st/algorithm/utils/src/hccl_verifier/checker.cc:50-100 pipeline;
// task_graph_generator.cc:51-65,144-153 Post/Wait matching and deadlock detection; mem_conflict_check/check_rank_mem.cc:509-696
// race check on fragments that are not ordered by happens-before; semantics_check/task_check_op_semantics.h:58-150 symbolic
// execution that tracks, for every output element, which (rank, input element) contributed), applied to the schedule IR of
// this library:
//   1. deadlock freedom   simulate all ranks' queues with counting notifies; no runnable task while some remain = deadlock
//   2. bounds             every access stays inside its buffer / scratch window
//   3. memory conflicts   vector clocks give happens-before; overlapping accesses with a write and no order are races
//   4. semantics          every output element ends up with exactly the contributor multiset the operator defines
#pragma once
#include <string>
#include <vector>
#include "../exec/op_param.h"
#include "../exec/plan.h"

namespace hccl {

struct CheckSpec {
    HcclCMDType op;
    uint32_t nranks;
    uint32_t elemSize;
    uint64_t count;                       // OpParam::count semantics
    uint32_t root;
    uint64_t cclBytes;
    std::vector<uint64_t> countMatrix;    // AlltoAllV(C): n*n (row = sender); AllGatherV / ReduceScatterV: n
    // point-to-point operators: Send / Receive move `count` elements from rank `root` to rank `peer`; BatchSendRecv is
    // checked as a bidirectional ring (every rank sends the first half of its input to rank + 1 and the second half to
    // rank - 1, and receives the matching halves into its output).
    uint32_t peer = 0;
    uint64_t mailboxBytes = 0;            // bytes of one mailbox slot (0 = unchecked)
    // ABS buffer references (BatchSendRecv items carry absolute addresses) are mapped back to the rank's input / output by range
    uint64_t absInputBase = 0, absOutputBase = 0;
    // zero-copy schedules: the callers' buffers are registered windows of the symmetric heap, so peers may address them
    bool registeredUserBuffers = false;
};
uint64_t CheckInputElems(const CheckSpec &s, uint32_t rank);
uint64_t CheckOutputElems(const CheckSpec &s, uint32_t rank);

struct SmLaunch;
// Schedule model of one SM / NVLS kernel launch (sm_models.cc).
HcclResult GenSmModelPlan(const std::vector<SmLaunch> &all, uint32_t me, uintptr_t inBase, uintptr_t outBase, uint32_t channels, Plan *out);

// plans[chunk][rank]; chunks run one after the other and share the symbolic memory.
HcclResult CheckPlans(const CheckSpec &spec, const std::vector<std::vector<Plan>> &plans, std::string *why);

}  // namespace hccl
