// Executors: compose templates / kernels into a complete operator run (chunk loop, resources, launch-plan cache).
//
// HCCL's executor taxonomy (reference: src/ops/op_common/executor/executor_v2_base.h:29-61 CalcAlgHierarchyInfo /
// CalcRes / Orchestrate; registry src/ops/op_common/executor/registry/coll_alg_v2_exec_registry.h:33-42,71):
//   Sole      one template on a flat rank list                         -> IrSoleExecutor, SmExecutor
//   Sequence  level 0, then level 1 (, then level 2) one after another -> IrSequenceExecutor (simulated multi-server)
//   Parallel  two shares of the data cross two levels in opposite orders, in pipelined steps -> IrParallelExecutor
//             (HCCL's Parallel and OmniPipe executors; the cut comes from slice_planner.cc)
//   P2P       send / recv / batch                                      -> P2pExecutor
// All share the outer chunk loop: maxCountPerLoop = what the scratch window can hold for the chosen template,
// iterate with a tail (reference: src/ops/all_reduce/executor/ins_v2_all_reduce_sole_executor.cc:125-176).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include "../core/comm.h"
#include "ir_templates.h"
#include "op_param.h"

namespace hccl {

struct AlgResourceRequest {          // what an executor needs before it can run (graph-mode resource queries)
    uint64_t scratchBytes = 0;
    uint32_t slaveStreams = 0;
    uint32_t notifyPerPeer = 0;
    uint32_t ctas = 0;
    uint64_t taskCount = 0;
};

class ExecutorBase {
public:
    virtual ~ExecutorBase() = default;
    virtual HcclResult CalcRes(Comm *c, const OpParam &p, AlgResourceRequest *req);
    virtual HcclResult Orchestrate(Comm *c, OpParam &p) = 0;
    void SetAlgName(const std::string &n) { algName_ = n; }
protected:
    std::string algName_;
};

class ExecutorRegistry {
public:
    static ExecutorRegistry &Instance();
    void Register(const std::string &algName, HcclCMDType op, std::function<ExecutorBase *()> factory);
    std::unique_ptr<ExecutorBase> Create(HcclCMDType op, const std::string &algName) const;
    std::vector<std::string> Names(HcclCMDType op) const;
    bool Has(HcclCMDType op, const std::string &algName) const;
private:
    std::map<std::pair<int, std::string>, std::function<ExecutorBase *()>> map_;
};
#define REGISTER_EXEC(name, op, cls) \
    static bool g_exec_##cls##_##op = (::hccl::ExecutorRegistry::Instance().Register(name, op, [] { return static_cast<::hccl::ExecutorBase *>(new cls()); }), true)

void RegisterBuiltinExecutors();   // idempotent; called by the dispatch core

// ---- launch-plan cache (HCCL: AIV launch cache / CCU fast launch; reference op_common.cc:357-412, hccl_aiv_utils.cc:713-800)
class PlanCache {
public:
    static PlanCache &Of(Comm *c);
    static void Drop(Comm *c);
    std::shared_ptr<const Plan> Find(const std::string &key);
    void Insert(const std::string &key, std::shared_ptr<const Plan> plan);
    size_t Size() const { return map_.size(); }
    static constexpr size_t kCapacity = 8192;      // entries; 20 % of the oldest are evicted when full
private:
    std::mutex mu_;
    std::map<std::string, std::shared_ptr<const Plan>> map_;
    std::deque<std::string> order_;
};

// Builds the per-chunk TemplateCtx list of an operator for a flat group (exposed for the offline checker).
struct ChunkCtx { TemplateCtx ctx; };
HcclResult BuildFlatChunks(const OpParam &p, uint32_t rank, uint32_t nranks, uint64_t cclBytes, const IrTemplate &tmpl,
                           std::vector<TemplateCtx> *chunks);
// Point-to-point plans (mailbox protocol).
HcclResult GenSendPlan(uint32_t me, uint32_t dst, uint64_t bytes, uint64_t mailboxBytes, Plan *p, size_t queue, BufRef src);
HcclResult GenRecvPlan(uint32_t me, uint32_t src, uint64_t bytes, uint64_t mailboxBytes, Plan *p, size_t queue, BufRef dst);
HcclResult GenBatchSendRecvPlan(uint32_t me, uint32_t nranks, const std::vector<HcclSendRecvItem> &items, uint64_t mailboxBytes,
                                Plan *p, std::vector<char *> *itemBufs);
// Multi-level plan for AllReduce / AllGather / ReduceScatter (whole op, no chunk loop).
HcclResult GenSequencePlan(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, Plan *plan);
// A call cut into the largest pieces whose plan fits the scratch. Each plan addresses the user buffers from the start of its piece
// (element `lo` of the vector, or of every rank's block for AllGather / ReduceScatter).
struct ChunkPlan { uint64_t lo, count; std::shared_ptr<Plan> plan; };
HcclResult GenSequenceChunkPlans(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, std::vector<ChunkPlan> *out);
HcclResult GenParallelChunkPlans(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, std::vector<ChunkPlan> *out);
// Broadcast, Reduce and Scatter on two levels; one plan per chunk of the message that fits the scratch.
HcclResult GenSequenceRootedPlans(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, std::vector<Plan> *plans);
// Two-level plan with both levels busy at once (parallel_executor.cc); slices = the planner's decision, if asked for.
struct SlicePlan;
HcclResult GenParallelPlan(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, Plan *plan, SlicePlan *slices = nullptr);

}  // namespace hccl
