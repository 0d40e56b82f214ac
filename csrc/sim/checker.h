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
};

// plans[chunk][rank]; chunks run one after the other and share the symbolic memory.
HcclResult CheckPlans(const CheckSpec &spec, const std::vector<std::vector<Plan>> &plans, std::string *why);

}  // namespace hccl
