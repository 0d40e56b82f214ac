#include "executor.h"
#include <algorithm>
#include <sstream>
#include "../common/dtype.h"
#include "../common/log.h"
#include "../kernels/launch.h"
#include "copy_engine.h"
#include "host_engine.h"

namespace hccl {

uint64_t OpParam::DataBytes() const
{
    uint64_t es = DataTypeSize(dtype);
    switch (opType) {
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: case HCCL_CMD_ALLGATHER_V: case HCCL_CMD_REDUCE_SCATTER_V: {
            uint64_t tot = 0;
            for (uint64_t c : (sendCounts.empty() ? recvCounts : sendCounts)) tot += c;
            return tot * es;
        }
        case HCCL_CMD_BATCH_SEND_RECV: {
            uint64_t tot = 0;
            for (auto &it : items) tot += it.count * DataTypeSize(it.dataType);
            return tot;
        }
        default: return count * es;
    }
}

// ------------------------------------------------------------------------------------------------ registry
ExecutorRegistry &ExecutorRegistry::Instance()
{
    static ExecutorRegistry r;
    return r;
}
void ExecutorRegistry::Register(const std::string &algName, HcclCMDType op, std::function<ExecutorBase *()> factory)
{
    map_[{(int)op, algName}] = std::move(factory);
}
std::unique_ptr<ExecutorBase> ExecutorRegistry::Create(HcclCMDType op, const std::string &algName) const
{
    auto it = map_.find({(int)op, algName});
    if (it == map_.end()) return nullptr;
    std::unique_ptr<ExecutorBase> e(it->second());
    e->SetAlgName(algName);
    return e;
}
std::vector<std::string> ExecutorRegistry::Names(HcclCMDType op) const
{
    std::vector<std::string> v;
    for (auto &kv : map_) if (kv.first.first == (int)op) v.push_back(kv.first.second);
    return v;
}
bool ExecutorRegistry::Has(HcclCMDType op, const std::string &algName) const { return map_.count({(int)op, algName}) != 0; }

HcclResult ExecutorBase::CalcRes(Comm *c, const OpParam &p, AlgResourceRequest *req)
{
    req->scratchBytes = std::min<uint64_t>(c->devComm.cclBytes, p.DataBytes() * c->nranks + (64u << 10));
    req->slaveStreams = 0;
    req->notifyPerPeer = 4;
    req->ctas = 0;
    req->taskCount = 1;
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ plan cache
namespace {
std::mutex g_pcMu;
std::map<Comm *, std::unique_ptr<PlanCache>> g_planCaches;
}
PlanCache &PlanCache::Of(Comm *c)
{
    std::lock_guard<std::mutex> lk(g_pcMu);
    auto &p = g_planCaches[c];
    if (!p) p.reset(new PlanCache());
    return *p;
}
void PlanCache::Drop(Comm *c)
{
    std::lock_guard<std::mutex> lk(g_pcMu);
    g_planCaches.erase(c);
}
std::shared_ptr<const Plan> PlanCache::Find(const std::string &key)
{
    std::lock_guard<std::mutex> lk(mu_);
    auto it = map_.find(key);
    return it == map_.end() ? nullptr : it->second;
}
void PlanCache::Insert(const std::string &key, std::shared_ptr<const Plan> plan)
{
    std::lock_guard<std::mutex> lk(mu_);
    if (map_.size() >= kCapacity) {
        size_t evict = kCapacity / 5;
        while (evict-- && !order_.empty()) { map_.erase(order_.front()); order_.pop_front(); }
    }
    if (map_.emplace(key, std::move(plan)).second) order_.push_back(key);
}

// ------------------------------------------------------------------------------------------------ chunking
static uint64_t Clamp(uint64_t total, uint64_t lo, uint64_t chunk) { return total <= lo ? 0 : std::min(chunk, total - lo); }

HcclResult BuildFlatChunks(const OpParam &p, uint32_t rank, uint32_t nranks, uint64_t cclBytes, const IrTemplate &tmpl,
                           std::vector<TemplateCtx> *chunks)
{
    uint32_t es = DataTypeSize(p.dtype);
    TemplateCtx base;
    base.group.resize(nranks);
    for (uint32_t r = 0; r < nranks; ++r) base.group[r] = r;
    base.me = rank;
    base.elemSize = es ? es : 1;
    base.cclOff = 0;
    base.cclBytes = cclBytes;
    base.root = p.root;
    base.inPlace = p.inputPtr == p.outputPtr;
    uint64_t maxCount = tmpl.maxCountPerLoop ? tmpl.maxCountPerLoop(nranks, base.elemSize, cclBytes) : 0;

    auto pushRange = [&](uint64_t total, const std::function<void(TemplateCtx &, uint64_t lo, uint64_t n)> &fill) {
        if (total == 0 || maxCount == 0) { TemplateCtx c = base; fill(c, 0, total); chunks->push_back(std::move(c)); return; }
        for (uint64_t lo = 0; lo < total; lo += maxCount) {
            TemplateCtx c = base;
            fill(c, lo, std::min(maxCount, total - lo));
            chunks->push_back(std::move(c));
        }
    };

    switch (p.opType) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_REDUCE:
            pushRange(p.count, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::INPUT, lo * es}; c.out = {BufKind::OUTPUT, lo * es};
            });
            break;
        case HCCL_CMD_BROADCAST:
            pushRange(p.count, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::OUTPUT, lo * es}; c.out = {BufKind::OUTPUT, lo * es}; c.inPlace = true;
            });
            break;
        case HCCL_CMD_ALLGATHER:
            pushRange(p.count, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::INPUT, lo * es}; c.out = {BufKind::OUTPUT, lo * es}; c.outStride = p.count * es;
                c.inPlace = (const char *)p.inputPtr == (const char *)p.outputPtr + (uint64_t)rank * p.count * es;
            });
            break;
        case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_SCATTER:
            pushRange(p.count, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::INPUT, lo * es}; c.out = {BufKind::OUTPUT, lo * es}; c.inStride = p.count * es; c.inPlace = false;
            });
            break;
        case HCCL_CMD_ALLTOALL:
            pushRange(p.count, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::INPUT, lo * es}; c.out = {BufKind::OUTPUT, lo * es};
                c.inStride = p.count * es; c.outStride = p.count * es; c.inPlace = false;
            });
            break;
        case HCCL_CMD_ALLGATHER_V: {
            if (p.recvCounts.size() != nranks || p.recvDispls.size() != nranks) return HCCL_E_PARA;
            uint64_t mx = *std::max_element(p.recvCounts.begin(), p.recvCounts.end());
            pushRange(mx, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::INPUT, lo * es}; c.out = {BufKind::OUTPUT, 0};
                c.recvBytes.resize(nranks); c.recvOff.resize(nranks);
                for (uint32_t r = 0; r < nranks; ++r) { c.recvBytes[r] = Clamp(p.recvCounts[r], lo, n) * es; c.recvOff[r] = (p.recvDispls[r] + lo) * es; }
                c.inPlace = false;
            });
            break;
        }
        case HCCL_CMD_REDUCE_SCATTER_V: {
            if (p.sendCounts.size() != nranks || p.sendDispls.size() != nranks) return HCCL_E_PARA;
            uint64_t mx = *std::max_element(p.sendCounts.begin(), p.sendCounts.end());
            pushRange(mx, [&](TemplateCtx &c, uint64_t lo, uint64_t n) {
                c.count = n; c.in = {BufKind::INPUT, 0}; c.out = {BufKind::OUTPUT, lo * es};
                c.sendBytes.resize(nranks); c.sendOff.resize(nranks);
                for (uint32_t r = 0; r < nranks; ++r) { c.sendBytes[r] = Clamp(p.sendCounts[r], lo, n) * es; c.sendOff[r] = (p.sendDispls[r] + lo) * es; }
                c.inPlace = false;
            });
            break;
        }
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: {
            if (p.sendCounts.size() != nranks || p.recvCounts.size() != nranks) return HCCL_E_PARA;
            TemplateCtx c = base;
            uint32_t esOut = DataTypeSize(p.outDtype);
            c.in = {BufKind::INPUT, 0}; c.out = {BufKind::OUTPUT, 0}; c.inPlace = false;
            c.sendBytes.resize(nranks); c.sendOff.resize(nranks); c.recvBytes.resize(nranks); c.recvOff.resize(nranks);
            for (uint32_t r = 0; r < nranks; ++r) {
                c.sendBytes[r] = p.sendCounts[r] * es; c.sendOff[r] = p.sendDispls[r] * es;
                c.recvBytes[r] = p.recvCounts[r] * esOut; c.recvOff[r] = p.recvDispls[r] * esOut;
            }
            chunks->push_back(std::move(c));
            break;
        }
        case HCCL_CMD_BARRIER: { TemplateCtx c = base; chunks->push_back(std::move(c)); break; }
        default: return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

static std::string PlanKey(const std::string &alg, const TemplateCtx &c, const OpParam &p)
{
    std::ostringstream os;
    os << alg << '|' << c.count << '|' << (int)p.dtype << '|' << (int)p.reduceOp << '|' << c.root << '|' << c.inPlace << '|' << c.in.off << '|'
       << c.out.off << '|' << c.inStride << '|' << c.outStride << '|' << c.N();
    for (auto *v : {&c.sendBytes, &c.sendOff, &c.recvBytes, &c.recvOff}) { os << '|'; for (uint64_t x : *v) os << x << ','; }
    return os.str();
}

// Runs one plan on the communicator's engine. Sim: queued on the worker. CUDA: issued on the stream.
static HcclResult RunPlan(Comm *c, const OpParam &p, std::shared_ptr<const Plan> plan, bool usesCclHalf)
{
    ExecBuffers bufs;
    bufs.in = (char *)p.inputPtr;
    bufs.out = (char *)p.outputPtr;
    bufs.cclHalf = usesCclHalf ? (uint32_t)(c->opSeq++ & 1) : 0;
    c->counters.chunkLoops++;
    if (c->backend == BackendKind::SIM) {
        c->worker->Enqueue([c, plan, bufs] { return HostEngineRun(c, *plan, bufs); });
        return HCCL_SUCCESS;
    }
    const bool isCollective = p.opType != HCCL_CMD_SEND && p.opType != HCCL_CMD_RECEIVE && p.opType != HCCL_CMD_BATCH_SEND_RECV;
    return CopyEngineRun(c, *plan, bufs, p.stream, isCollective);
}

// ------------------------------------------------------------------------------------------------ IR sole executor
class IrSoleExecutor : public ExecutorBase {
public:
    HcclResult Orchestrate(Comm *c, OpParam &p) override
    {
        RegisterBuiltinIrTemplates();
        const IrTemplate *t = IrTemplateRegistry::Instance().Find(algName_);
        if (!t) { HCCL_ERROR("no IR template named %s", algName_.c_str()); return HCCL_E_NOT_FOUND; }
        std::vector<TemplateCtx> chunks;
        CHK_RET(BuildFlatChunks(p, c->rank, c->nranks, c->devComm.cclBytes, *t, &chunks));
        PlanCache &cache = PlanCache::Of(c);
        for (const TemplateCtx &ctx : chunks) {
            std::string key = PlanKey(algName_, ctx, p);
            std::shared_ptr<const Plan> plan = cache.Find(key);
            if (plan) c->counters.planCacheHits++;
            else {
                c->counters.planCacheMisses++;
                auto fresh = std::make_shared<Plan>();
                fresh->dtype = p.dtype;
                fresh->op = p.reduceOp;
                CHK_RET(t->gen(ctx, fresh.get()));
                plan = fresh;
                cache.Insert(key, plan);
            }
            CHK_RET(RunPlan(c, p, plan, true));
        }
        return HCCL_SUCCESS;
    }
    HcclResult CalcRes(Comm *c, const OpParam &p, AlgResourceRequest *req) override
    {
        RegisterBuiltinIrTemplates();
        const IrTemplate *t = IrTemplateRegistry::Instance().Find(algName_);
        if (!t) return HCCL_E_NOT_FOUND;
        std::vector<TemplateCtx> chunks;
        CHK_RET(BuildFlatChunks(p, c->rank, c->nranks, c->devComm.cclBytes, *t, &chunks));
        req->taskCount = 0;
        for (auto &ctx : chunks) { Plan pl; CHK_RET(t->gen(ctx, &pl)); req->taskCount += pl.TaskCount(); }
        req->scratchBytes = c->devComm.cclBytes;
        req->slaveStreams = 0;
        req->notifyPerPeer = kNotifySlots;
        return HCCL_SUCCESS;
    }
};

// ------------------------------------------------------------------------------------------------ p2p plans
HcclResult GenSendPlan(uint32_t, uint32_t dst, uint64_t bytes, uint64_t W, Plan *p, size_t queue, BufRef src)
{
    p->EnsureQueues(queue + 1);
    auto &q = p->queues[queue];
    uint64_t rounds = (bytes + W - 1) / W;
    for (uint64_t k = 0; k < rounds; ++k) {
        if (k >= 2) q.push_back(Task{TaskType::WAIT, dst, 9, {}, {}, 0});
        uint64_t len = std::min(W, bytes - k * W);
        BufRef s = src;
        s.off += k * W;
        q.push_back(Task{TaskType::LOCAL_COPY, 0, 0, BufRef{BufKind::MAILBOX, ((uint64_t)dst * 2 + (k & 1)) * W}, s, len});
        q.push_back(Task{TaskType::POST, dst, 8, {}, {}, 0});
    }
    for (uint64_t k = 0; k < std::min<uint64_t>(rounds, 2); ++k) q.push_back(Task{TaskType::WAIT, dst, 9, {}, {}, 0});
    return HCCL_SUCCESS;
}

HcclResult GenRecvPlan(uint32_t me, uint32_t src, uint64_t bytes, uint64_t W, Plan *p, size_t queue, BufRef dst)
{
    p->EnsureQueues(queue + 1);
    auto &q = p->queues[queue];
    uint64_t rounds = (bytes + W - 1) / W;
    for (uint64_t k = 0; k < rounds; ++k) {
        q.push_back(Task{TaskType::WAIT, src, 8, {}, {}, 0});
        uint64_t len = std::min(W, bytes - k * W);
        BufRef d = dst;
        d.off += k * W;
        q.push_back(Task{TaskType::READ, src, 0, d, BufRef{BufKind::MAILBOX, ((uint64_t)me * 2 + (k & 1)) * W}, len});
        q.push_back(Task{TaskType::POST, src, 9, {}, {}, 0});
    }
    return HCCL_SUCCESS;
}

// Items are ordered the way HCCL orders them for deadlock freedom (sends by descending, receives by ascending
// ring distance, ties by count then dtype; reference: ins_v2_batch_send_recv_executor.cc:106-206), self pairs
// are matched and turned into local copies (:80-104), and every (peer, direction) pair gets its own queue so
// unrelated pairs never wait for each other.
HcclResult GenBatchSendRecvPlan(uint32_t me, uint32_t nranks, const std::vector<HcclSendRecvItem> &items, uint64_t W, Plan *p,
                                std::vector<char *> *)
{
    std::vector<HcclSendRecvItem> sends, recvs, selfS, selfR;
    for (auto &it : items) {
        if (it.remoteRank >= nranks) return HCCL_E_PARA;
        if (it.remoteRank == me) (it.sendRecvType == HCCL_SEND ? selfS : selfR).push_back(it);
        else (it.sendRecvType == HCCL_SEND ? sends : recvs).push_back(it);
    }
    if (selfS.size() != selfR.size()) { HCCL_ERROR("BatchSendRecv: %zu self sends but %zu self receives", selfS.size(), selfR.size()); return HCCL_E_PARA; }
    p->EnsureQueues(1);
    for (size_t i = 0; i < selfS.size(); ++i) {
        uint64_t sb = selfS[i].count * DataTypeSize(selfS[i].dataType), rb = selfR[i].count * DataTypeSize(selfR[i].dataType);
        if (sb != rb) { HCCL_ERROR("BatchSendRecv: self pair %zu size mismatch (%llu vs %llu bytes)", i, (unsigned long long)sb, (unsigned long long)rb); return HCCL_E_PARA; }
        if (sb) p->queues[0].push_back(Task{TaskType::LOCAL_COPY, 0, 0, BufRef{BufKind::ABS, (uint64_t)(uintptr_t)selfR[i].buf},
                                            BufRef{BufKind::ABS, (uint64_t)(uintptr_t)selfS[i].buf}, sb});
    }
    auto keyOf = [&](uint32_t remote) { return remote <= me ? remote + nranks : remote; };
    std::stable_sort(sends.begin(), sends.end(), [&](const HcclSendRecvItem &a, const HcclSendRecvItem &b) { return keyOf(a.remoteRank) > keyOf(b.remoteRank); });
    std::stable_sort(recvs.begin(), recvs.end(), [&](const HcclSendRecvItem &a, const HcclSendRecvItem &b) { return keyOf(a.remoteRank) < keyOf(b.remoteRank); });
    std::map<std::pair<uint32_t, int>, size_t> queueOf;
    auto queueFor = [&](uint32_t peer, int dir) {
        auto it = queueOf.find({peer, dir});
        if (it != queueOf.end()) return it->second;
        size_t q = queueOf.size() + 1;
        queueOf[{peer, dir}] = q;
        return q;
    };
    for (auto &it : sends) CHK_RET(GenSendPlan(me, it.remoteRank, it.count * DataTypeSize(it.dataType), W, p, queueFor(it.remoteRank, 0), BufRef{BufKind::ABS, (uint64_t)(uintptr_t)it.buf}));
    for (auto &it : recvs) CHK_RET(GenRecvPlan(me, it.remoteRank, it.count * DataTypeSize(it.dataType), W, p, queueFor(it.remoteRank, 1), BufRef{BufKind::ABS, (uint64_t)(uintptr_t)it.buf}));
    return HCCL_SUCCESS;
}

class IrP2pExecutor : public ExecutorBase {
public:
    HcclResult Orchestrate(Comm *c, OpParam &p) override
    {
        auto plan = std::make_shared<Plan>();
        plan->dtype = p.dtype;
        uint64_t W = c->devComm.mailboxBytes;
        if (p.opType == HCCL_CMD_SEND) CHK_RET(GenSendPlan(c->rank, p.peer, p.DataBytes(), W, plan.get(), 0, BufRef{BufKind::INPUT, 0}));
        else if (p.opType == HCCL_CMD_RECEIVE) CHK_RET(GenRecvPlan(c->rank, p.peer, p.DataBytes(), W, plan.get(), 0, BufRef{BufKind::OUTPUT, 0}));
        else CHK_RET(GenBatchSendRecvPlan(c->rank, c->nranks, p.items, W, plan.get(), nullptr));
        return RunPlan(c, p, plan, false);
    }
};

// ------------------------------------------------------------------------------------------------ sequence executor
namespace {
struct LevelGroup { std::vector<uint32_t> ranks; uint32_t me; };

const IrTemplate *Tmpl(const char *name)
{
    RegisterBuiltinIrTemplates();
    return IrTemplateRegistry::Instance().Find(name);
}
uint64_t Al(uint64_t v) { return (v + 511) / 512 * 512; }
}  // namespace

HcclResult GenSequencePlan(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, Plan *plan)
{
    AlgHierarchyInfo h;
    CHK_RET(TopoMatch(topo, TopoMatchKind::MULTI_LEVEL, &h));
    if (h.levelRanks.size() < 2) return HCCL_E_NOT_SUPPORT;
    uint32_t es = DataTypeSize(p.dtype);
    uint32_t n0 = (uint32_t)h.levelRanks[0].size(), me0 = h.myIndex[0];
    plan->dtype = p.dtype;
    plan->op = p.reduceOp;
    auto baseCtx = [&](uint32_t level) {
        TemplateCtx c;
        c.group = h.levelRanks[level];
        c.me = h.myIndex[level];
        c.elemSize = es;
        return c;
    };
    if (p.opType == HCCL_CMD_ALLREDUCE) {
        // level 0 reduce-scatter (uneven slices) -> all-reduce of my slice on every upper level -> level 0 all-gather
        uint64_t per = (p.count + n0 - 1) / n0;
        std::vector<uint64_t> len(n0), off(n0);
        for (uint32_t j = 0; j < n0; ++j) { off[j] = std::min(p.count, per * j) * es; len[j] = Clamp(p.count, per * j, per) * es; }
        uint64_t W0 = Al(per * es) * n0 + 4096;
        uint64_t upperCount = len[me0] / es;
        uint64_t W1 = 0;
        for (size_t l = 1; l < h.levelRanks.size(); ++l) W1 = std::max<uint64_t>(W1, 4 * Al(per * es) + 65536);
        uint64_t need = W0 + W1 * (h.levelRanks.size() - 1) + Al(per * es) + 4096;
        if (need > cclBytes) { HCCL_ERROR("sequence all-reduce needs %llu bytes of scratch, have %llu (raise HCCL_BUFFSIZE)", (unsigned long long)need, (unsigned long long)cclBytes); return HCCL_E_MEMORY; }
        TemplateCtx a = baseCtx(0);
        a.in = {BufKind::INPUT, 0}; a.out = {BufKind::OUTPUT, off[me0]};
        a.sendBytes = len; a.sendOff = off; a.cclOff = 0; a.cclBytes = W0;
        CHK_RET(Tmpl("InsReduceScatterVMesh1D")->gen(a, plan));
        uint64_t win = W0;
        for (size_t l = 1; l < h.levelRanks.size(); ++l) {
            TemplateCtx b = baseCtx((uint32_t)l);
            b.count = upperCount; b.in = {BufKind::OUTPUT, off[me0]}; b.out = b.in; b.inPlace = true; b.cclOff = win; b.cclBytes = W1;
            if (upperCount) CHK_RET(Tmpl("InsAllReduceNHR")->gen(b, plan));
            win += W1;
        }
        TemplateCtx g = baseCtx(0);
        g.in = {BufKind::OUTPUT, off[me0]}; g.out = {BufKind::OUTPUT, 0}; g.recvBytes = len; g.recvOff = off; g.cclOff = win; g.cclBytes = Al(per * es) + 4096;
        CHK_RET(Tmpl("InsAllGatherVMesh1D")->gen(g, plan));
        return HCCL_SUCCESS;
    }
    // AllGather and ReduceScatter are written for two levels: everything above the server counts as one
    if (h.levelRanks.size() > 2) CHK_RET(TopoMatch(topo, TopoMatchKind::TWO_LEVEL, &h));
    if (h.levelRanks.size() != 2) return HCCL_E_NOT_SUPPORT;
    const auto &g1 = h.levelRanks[1];
    uint32_t n1 = (uint32_t)g1.size();
    uint64_t B = p.count * es, S = Al(B);
    const uint64_t T = (p.blockStride ? p.blockStride : p.count) * es;       // bytes between the per-rank blocks of the user buffers
    if (p.opType == HCCL_CMD_ALLGATHER) {
        // level 1: gather my block across servers; level 0: one gather per server's block set
        if (S * (1 + n1) + 8192 > cclBytes) return HCCL_E_MEMORY;
        TemplateCtx a = baseCtx(1);
        a.in = {BufKind::INPUT, 0}; a.out = {BufKind::OUTPUT, 0}; a.cclOff = 0; a.cclBytes = S + 4096;
        a.recvBytes.assign(n1, B); a.recvOff.resize(n1);
        for (uint32_t k = 0; k < n1; ++k) a.recvOff[k] = (uint64_t)g1[k] * T;
        CHK_RET(Tmpl("InsAllGatherVMesh1D")->gen(a, plan));
        for (uint32_t s = 0; s < n1; ++s) {
            // the server that g1[s] belongs to: its level-0 group is {g1[s] - me0 + j}
            uint32_t base = g1[s] - me0;
            TemplateCtx b = baseCtx(0);
            b.in = {BufKind::OUTPUT, (uint64_t)(base + me0) * T}; b.out = {BufKind::OUTPUT, 0};
            b.cclOff = S + 4096 + (uint64_t)s * S; b.cclBytes = S;
            b.recvBytes.assign(n0, B); b.recvOff.resize(n0);
            for (uint32_t j = 0; j < n0; ++j) b.recvOff[j] = (uint64_t)(base + j) * T;
            CHK_RET(Tmpl("InsAllGatherVMesh1D")->gen(b, plan));
        }
        return HCCL_SUCCESS;
    }
    if (p.opType == HCCL_CMD_REDUCE_SCATTER) {
        // level 0: per server-block reduce-scatter into a work area; level 1: reduce-scatter of the n1 partials
        uint64_t workOff = 0, win0 = Al(S * n1 + 4096), per0 = S * n0 + 4096, win1 = win0 + per0 * n1;
        if (win1 + S * n1 + 4096 > cclBytes) return HCCL_E_MEMORY;
        for (uint32_t s = 0; s < n1; ++s) {
            uint32_t base = g1[s] - me0;
            TemplateCtx a = baseCtx(0);
            a.in = {BufKind::INPUT, 0}; a.out = {BufKind::CCL, workOff + (uint64_t)s * S};
            a.sendBytes.assign(n0, B); a.sendOff.resize(n0);
            for (uint32_t j = 0; j < n0; ++j) a.sendOff[j] = (uint64_t)(base + j) * T;
            a.cclOff = win0 + per0 * s; a.cclBytes = per0;
            CHK_RET(Tmpl("InsReduceScatterVMesh1D")->gen(a, plan));
        }
        TemplateCtx b = baseCtx(1);
        b.count = p.count; b.in = {BufKind::CCL, workOff}; b.inStride = S; b.out = {BufKind::OUTPUT, 0}; b.cclOff = win1; b.cclBytes = S * n1 + 4096;
        CHK_RET(Tmpl("InsReduceScatterMesh1D")->gen(b, plan));
        return HCCL_SUCCESS;
    }
    return HCCL_E_NOT_SUPPORT;
}

// Rooted operators (and the barrier) on two levels. The root's column (the ranks at the root's position in every server) is the only
// level-1 group that carries data: Broadcast crosses the servers once and fans out inside each one; Reduce sums inside
// every server onto the root's position and then across the servers (server order, so the bits do not depend on timing);
// Scatter moves each server's blocks to that server's member of the column, which hands them out. A message that does
// not fit the scratch is cut into chunks, one plan each; every template used here ends in a barrier of its group, so a
// plan may reuse the scratch half of the plan before the previous one.
// HCCL builds the same shapes as its sequence executors for the rooted operators (reference:
// src/ops/broadcast/executor/ins_v2_broadcast_sequence_executor.cc, src/ops/reduce/executor/ins_v2_reduce_sequence_executor.cc,
// src/ops/scatter/executor/ins_v2_scatter_sequence_executor.cc).
HcclResult GenSequenceRootedPlans(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, std::vector<Plan> *plans)
{
    AlgHierarchyInfo h;
    CHK_RET(TopoMatch(topo, TopoMatchKind::TWO_LEVEL, &h));
    if (h.levelRanks.size() != 2) return HCCL_E_NOT_SUPPORT;
    const auto &g0 = h.levelRanks[0], &g1 = h.levelRanks[1];
    const uint32_t n0 = (uint32_t)g0.size(), n1 = (uint32_t)g1.size(), me0 = h.myIndex[0], es = DataTypeSize(p.dtype);
    // servers hold consecutive ranks, n0 each: server s starts at rank s * n0
    for (uint32_t s = 0; s < n1; ++s) if (g1[s] != s * n0 + me0) return HCCL_E_NOT_SUPPORT;
    if (p.opType == HCCL_CMD_BARRIER) {
        // inside the server, then along my column: every member of the column has seen its whole server arrive
        // (reference: src/ops/barrier/executor/ins_v2_barrier_sequence_executor.cc)
        Plan pl;
        pl.dtype = p.dtype;
        pl.EnsureQueues(1);
        for (uint32_t level = 0; level < 2; ++level) {
            TemplateCtx b;
            b.group = h.levelRanks[level];
            b.me = h.myIndex[level];
            b.elemSize = es;
            CHK_RET(Tmpl("InsBarrierMesh1D")->gen(b, &pl));
        }
        plans->clear();
        plans->push_back(std::move(pl));
        return HCCL_SUCCESS;
    }
    if (p.root >= n0 * n1) return HCCL_E_PARA;
    const uint32_t rootServer = p.root / n0, rootPos = p.root % n0;
    const bool inColumn = me0 == rootPos;

    // Two forms. The column form moves the whole message through the root's column (two hops; small messages). The spread form
    // gives every column a share: Broadcast scatters slices inside the root's server, broadcasts each along its column and gathers
    // inside every server; Reduce is its mirror (reduce-scatter inside every server, reduce along the columns, gather at the root);
    // Scatter hands each member of the root's server the blocks of its column and scatters along the columns. The root's link to
    // the other servers then carries 1 / n0 of the bytes. Both forms of Reduce sum in the same order (ranks of a server, then
    // servers), so the bits do not depend on the form.
    const uint64_t kSpreadBytes = 256u << 10;
    const bool spread = n0 > 1 && n1 > 1 && (p.opType == HCCL_CMD_SCATTER || p.count * es >= kSpreadBytes);
    // scratch per chunk, in units of the aligned piece S: column form Broadcast 2 S, Reduce (1 + n0 + n1) S, Scatter (2 n0 + n1) S with
    // S = Al(c * es); spread form Broadcast (n0 + 2) S, Reduce (n0 + n1 + 3) S with S = Al(ceil(c / n0) * es), Scatter (2 n1 + n0) S
    uint64_t units;
    if (p.opType == HCCL_CMD_BROADCAST) units = spread ? n0 + 2 : 2;
    else if (p.opType == HCCL_CMD_REDUCE) units = spread ? n0 + n1 + 3 : 1 + n0 + n1;
    else units = spread ? 2 * n1 + n0 : 2 * n0 + n1;
    const uint64_t slack = 4 * 4096;
    if (cclBytes < slack + units * 512) return HCCL_E_MEMORY;
    uint64_t maxCount = (cclBytes - slack) / units / 512 * 512 / es;
    if (spread && p.opType != HCCL_CMD_SCATTER) maxCount *= n0;                 // the piece is a slice of the chunk
    if (maxCount == 0) return HCCL_E_MEMORY;
    auto ctxOf = [&](uint32_t level) {
        TemplateCtx c;
        c.group = h.levelRanks[level];
        c.me = h.myIndex[level];
        c.elemSize = es;
        return c;
    };
    const bool inRootServer = h.myIndex[1] == rootServer;
    const bool isRoot = inColumn && inRootServer;
    plans->clear();
    for (uint64_t lo = 0; lo < std::max<uint64_t>(p.count, 1); lo += maxCount) {
        const uint64_t cnt = std::min(maxCount, p.count - lo), S = Al(cnt * es);
        Plan pl;
        pl.dtype = p.dtype;
        pl.op = p.reduceOp;
        pl.EnsureQueues(1);
        if (cnt == 0) { plans->push_back(std::move(pl)); break; }
        // slices of the chunk over the positions of a server (spread forms of Broadcast and Reduce)
        const uint64_t per = (cnt + n0 - 1) / n0, Sa = Al(per * es);
        std::vector<uint64_t> len(n0), off(n0);
        for (uint32_t k = 0; k < n0; ++k) { off[k] = std::min(cnt, per * k) * es; len[k] = Clamp(cnt, per * k, per) * es; }
        const char *bcast = nullptr;
        auto bcastFor = [](uint64_t bytes) { return bytes >= (64u << 10) ? "InsBroadcastMesh1DTwoShot" : "InsBroadcastMesh1DOneShot"; };
        if (p.opType == HCCL_CMD_BROADCAST && spread) {
            const uint64_t winB = n0 * Sa + 4096, winC = winB + Sa + 4096;
            if (inRootServer) {
                TemplateCtx a = ctxOf(0);
                a.root = rootPos; a.in = {BufKind::OUTPUT, lo * es}; a.out = {BufKind::OUTPUT, lo * es + off[me0]};
                a.sendBytes = len; a.sendOff = off; a.inPlace = true; a.cclOff = 0; a.cclBytes = winB;
                CHK_RET(Tmpl("InsScatterMesh1D")->gen(a, &pl));
            }
            if (len[me0]) {
                TemplateCtx b = ctxOf(1);
                b.count = len[me0] / es; b.root = rootServer; b.in = b.out = {BufKind::OUTPUT, lo * es + off[me0]}; b.inPlace = true;
                b.cclOff = winB; b.cclBytes = Sa + 4096;
                CHK_RET(Tmpl(bcastFor(len[me0]))->gen(b, &pl));
            }
            TemplateCtx g = ctxOf(0);
            g.in = {BufKind::OUTPUT, lo * es + off[me0]}; g.out = {BufKind::OUTPUT, lo * es}; g.recvBytes = len; g.recvOff = off;
            g.cclOff = winC; g.cclBytes = Sa + 4096;
            CHK_RET(Tmpl("InsAllGatherVMesh1D")->gen(g, &pl));
        } else if (p.opType == HCCL_CMD_BROADCAST) {
            bcast = bcastFor(cnt * es);
            if (inColumn && n1 > 1) {
                TemplateCtx a = ctxOf(1);
                a.count = cnt; a.root = rootServer; a.in = a.out = {BufKind::OUTPUT, lo * es}; a.inPlace = true; a.cclOff = 0; a.cclBytes = S + 4096;
                CHK_RET(Tmpl(bcast)->gen(a, &pl));
            }
            TemplateCtx b = ctxOf(0);
            b.count = cnt; b.root = rootPos; b.in = b.out = {BufKind::OUTPUT, lo * es}; b.inPlace = true; b.cclOff = S + 4096; b.cclBytes = S + 4096;
            CHK_RET(Tmpl(bcast)->gen(b, &pl));
        } else if (p.opType == HCCL_CMD_REDUCE && spread) {
            // [0, Sa): my slice summed over my server; [Sa, 2 Sa): summed over all servers (members of the root's server)
            const uint64_t winA = 2 * Sa, winB = winA + n0 * Sa, winC = winB + n1 * Sa + 4096;
            TemplateCtx a = ctxOf(0);
            a.in = {BufKind::INPUT, lo * es}; a.out = {BufKind::CCL, 0}; a.sendBytes = len; a.sendOff = off; a.cclOff = winA; a.cclBytes = n0 * Sa;
            CHK_RET(Tmpl("InsReduceScatterVMesh1D")->gen(a, &pl));
            if (len[me0]) {
                TemplateCtx b = ctxOf(1);
                b.count = len[me0] / es; b.root = rootServer; b.in = {BufKind::CCL, 0}; b.out = {BufKind::CCL, Sa}; b.cclOff = winB; b.cclBytes = n1 * Sa + 4096;
                CHK_RET(Tmpl("ReduceMesh1D")->gen(b, &pl));
            }
            if (inRootServer) {
                TemplateCtx g = ctxOf(0);
                g.root = rootPos; g.in = {BufKind::CCL, Sa}; g.out = {BufKind::OUTPUT, lo * es}; g.recvBytes = len; g.recvOff = off;
                g.cclOff = winC; g.cclBytes = Sa + 4096;
                CHK_RET(Tmpl("InsGatherMesh1D")->gen(g, &pl));
            }
        } else if (p.opType == HCCL_CMD_REDUCE) {
            const uint64_t win0 = S, win1 = win0 + n0 * S + 4096;
            TemplateCtx a = ctxOf(0);
            a.count = cnt; a.root = rootPos; a.in = {BufKind::INPUT, lo * es}; a.out = {BufKind::CCL, 0}; a.cclOff = win0; a.cclBytes = n0 * S + 4096;
            if (n1 == 1 && isRoot) a.out = {BufKind::OUTPUT, lo * es};
            CHK_RET(Tmpl("ReduceMesh1D")->gen(a, &pl));
            if (inColumn && n1 > 1) {
                TemplateCtx b = ctxOf(1);
                b.count = cnt; b.root = rootServer; b.in = {BufKind::CCL, 0}; b.out = isRoot ? BufRef{BufKind::OUTPUT, lo * es} : BufRef{BufKind::CCL, 0};
                b.cclOff = win1; b.cclBytes = n1 * S + 4096;
                CHK_RET(Tmpl("ReduceMesh1D")->gen(b, &pl));
            }
        } else if (p.opType == HCCL_CMD_SCATTER && spread) {
            // stage area: the blocks of my column, one per server, S apart; filled inside the root's server by one scatter per server
            const uint64_t win0 = n1 * S, win1 = win0 + n0 * S + 4096;
            if (inRootServer) {
                for (uint32_t sv = 0; sv < n1; ++sv) {
                    TemplateCtx a = ctxOf(0);
                    a.count = cnt; a.root = rootPos;
                    a.in = {BufKind::INPUT, ((uint64_t)sv * n0 * p.count + lo) * es}; a.inStride = p.count * es;
                    a.out = {BufKind::CCL, (uint64_t)sv * S}; a.cclOff = win0; a.cclBytes = n0 * S + 4096;
                    CHK_RET(Tmpl("InsScatterMesh1D")->gen(a, &pl));
                }
            }
            TemplateCtx b = ctxOf(1);
            b.count = cnt; b.root = rootServer; b.in = {BufKind::CCL, 0}; b.inStride = S; b.out = {BufKind::OUTPUT, lo * es}; b.cclOff = win1; b.cclBytes = n1 * S + 4096;
            CHK_RET(Tmpl("InsScatterMesh1D")->gen(b, &pl));
        } else if (p.opType == HCCL_CMD_SCATTER) {
            // one level is trivial. Stage area: the n0 blocks of my server, S apart; filled over level 1 by one scatter per position
            const uint64_t win1 = n0 * S, win0 = win1 + n1 * S + 4096;
            if (inColumn) {
                for (uint32_t k = 0; k < n0; ++k) {
                    TemplateCtx a = ctxOf(1);
                    a.count = cnt; a.root = rootServer;
                    a.in = {BufKind::INPUT, ((uint64_t)k * p.count + lo) * es}; a.inStride = (uint64_t)n0 * p.count * es;
                    a.out = {BufKind::CCL, (uint64_t)k * S}; a.cclOff = win1; a.cclBytes = n1 * S + 4096;
                    if (n1 > 1) CHK_RET(Tmpl("InsScatterMesh1D")->gen(a, &pl));
                    else pl.queues[0].push_back(Task{TaskType::LOCAL_COPY, 0, 0, a.out, a.in, cnt * es});
                }
            }
            TemplateCtx b = ctxOf(0);
            b.count = cnt; b.root = rootPos; b.in = {BufKind::CCL, 0}; b.inStride = S; b.out = {BufKind::OUTPUT, lo * es}; b.cclOff = win0; b.cclBytes = n0 * S + 4096;
            CHK_RET(Tmpl("InsScatterMesh1D")->gen(b, &pl));
        } else {
            return HCCL_E_NOT_SUPPORT;
        }
        plans->push_back(std::move(pl));
    }
    return HCCL_SUCCESS;
}

class IrSequenceRootedExecutor : public ExecutorBase {
public:
    HcclResult Orchestrate(Comm *c, OpParam &p) override
    {
        std::vector<Plan> plans;
        CHK_RET(GenSequenceRootedPlans(p, c->topo, c->devComm.cclBytes, &plans));
        for (Plan &pl : plans) CHK_RET(RunPlan(c, p, std::make_shared<Plan>(std::move(pl)), true));
        return HCCL_SUCCESS;
    }
};

// The chunk loop of the multi-level executors: the largest piece of the call whose plan fits the scratch is found by halving (the
// answer depends on the topology and the scratch size only, so every rank finds the same one), then one plan runs per piece. A piece
// of AllGather / ReduceScatter keeps the block stride of the whole call. HCCL's executors share the same outer loop (reference:
// src/ops/all_reduce/executor/ins_v2_all_reduce_sole_executor.cc:125-176).
template <class Gen>
static HcclResult GenMultiLevelChunks(const OpParam &p, uint64_t cclBytes, Gen gen, std::vector<ChunkPlan> *out)
{
    out->clear();
    // per: the size that fitted last. A later piece may have to be smaller still (the parallel planner cuts a short tail into fewer,
    // larger steps), so every piece is tried on its own.
    uint64_t per = p.count;
    for (uint64_t lo = 0; lo < p.count;) {
        uint64_t cnt = std::min(per, p.count - lo);
        for (;;) {
            OpParam q = p;
            q.count = cnt;
            q.blockStride = p.count;
            auto plan = std::make_shared<Plan>();
            LogPushMute();                         // "does not fit" is an answer here, not an error
            HcclResult r = gen(q, plan.get());
            LogPopMute();
            if (r == HCCL_SUCCESS) { out->push_back(ChunkPlan{lo, cnt, plan}); break; }
            if (r != HCCL_E_MEMORY || cnt <= 1024) {
                if (r == HCCL_E_MEMORY) HCCL_ERROR("%s: not even 1024 elements fit the scratch of %llu bytes (raise HCCL_BUFFSIZE)", p.algName.c_str(), (unsigned long long)cclBytes);
                return r;
            }
            cnt = (cnt / 2 + 127) / 128 * 128;
        }
        per = cnt;
        lo += cnt;
    }
    return HCCL_SUCCESS;
}

HcclResult GenSequenceChunkPlans(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, std::vector<ChunkPlan> *out)
{
    return GenMultiLevelChunks(p, cclBytes, [&](const OpParam &q, Plan *plan) { return GenSequencePlan(q, topo, cclBytes, plan); }, out);
}
HcclResult GenParallelChunkPlans(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, std::vector<ChunkPlan> *out)
{
    return GenMultiLevelChunks(p, cclBytes, [&](const OpParam &q, Plan *plan) { return GenParallelPlan(q, topo, cclBytes, plan); }, out);
}

// Runs the pieces: each plan addresses the user buffers from the start of its piece.
static HcclResult RunChunkPlans(Comm *c, const OpParam &p, const std::vector<ChunkPlan> &chunks)
{
    const uint32_t es = DataTypeSize(p.dtype);
    for (const ChunkPlan &ch : chunks) {
        OpParam q = p;
        q.count = ch.count;
        q.blockStride = p.count;
        q.inputPtr = p.inputPtr ? (const char *)p.inputPtr + ch.lo * es : nullptr;
        q.outputPtr = p.outputPtr ? (char *)p.outputPtr + ch.lo * es : nullptr;
        CHK_RET(RunPlan(c, q, ch.plan, true));
    }
    return HCCL_SUCCESS;
}

class IrSequenceExecutor : public ExecutorBase {
public:
    HcclResult Orchestrate(Comm *c, OpParam &p) override
    {
        std::vector<ChunkPlan> chunks;
        CHK_RET(GenSequenceChunkPlans(p, c->topo, c->devComm.cclBytes, &chunks));
        return RunChunkPlans(c, p, chunks);
    }
};

class IrParallelExecutor : public ExecutorBase {
public:
    HcclResult Orchestrate(Comm *c, OpParam &p) override
    {
        if (c->backend != BackendKind::SIM) {
            HCCL_ERROR("%s: schedules with several queues run on the host engine only", algName_.c_str());
            return HCCL_E_NOT_SUPPORT;
        }
        std::vector<ChunkPlan> chunks;
        CHK_RET(GenParallelChunkPlans(p, c->topo, c->devComm.cclBytes, &chunks));
        return RunChunkPlans(c, p, chunks);
    }
};

// ------------------------------------------------------------------------------------------------ SM / NVLS executor
class SmExecutor : public ExecutorBase {
public:
    HcclResult Orchestrate(Comm *c, OpParam &p) override
    {
        if (c->backend != BackendKind::CUDA) return HCCL_E_UNAVAIL;
        return SmOrchestrate(c, p, algName_);
    }
    HcclResult CalcRes(Comm *c, const OpParam &p, AlgResourceRequest *req) override
    {
        ExecutorBase::CalcRes(c, p, req);
        req->ctas = SmDefaultCtas(p.opType, algName_, p.DataBytes(), c->nranks);
        return HCCL_SUCCESS;
    }
};

void RegisterBuiltinExecutors()
{
    static std::once_flag once;
    std::call_once(once, [] {
        RegisterBuiltinIrTemplates();
        auto &R = ExecutorRegistry::Instance();
        for (int op = 1; op < (int)HCCL_CMD_MAX; ++op)
            for (auto &nm : IrTemplateRegistry::Instance().Names((HcclCMDType)op))
                R.Register(nm, (HcclCMDType)op, [] { return static_cast<ExecutorBase *>(new IrSoleExecutor()); });
        R.Register("InsSend", HCCL_CMD_SEND, [] { return static_cast<ExecutorBase *>(new IrP2pExecutor()); });
        R.Register("InsRecv", HCCL_CMD_RECEIVE, [] { return static_cast<ExecutorBase *>(new IrP2pExecutor()); });
        R.Register("InsBatchSendRecv", HCCL_CMD_BATCH_SEND_RECV, [] { return static_cast<ExecutorBase *>(new IrP2pExecutor()); });
        R.Register("InsAllReduceSequenceMesh1DNhr", HCCL_CMD_ALLREDUCE, [] { return static_cast<ExecutorBase *>(new IrSequenceExecutor()); });
        R.Register("InsAllGatherSequenceNhrMesh1D", HCCL_CMD_ALLGATHER, [] { return static_cast<ExecutorBase *>(new IrSequenceExecutor()); });
        R.Register("InsReduceScatterSequenceMesh1DNhr", HCCL_CMD_REDUCE_SCATTER, [] { return static_cast<ExecutorBase *>(new IrSequenceExecutor()); });
        R.Register("InsBroadcastSequenceMesh1DMesh1D", HCCL_CMD_BROADCAST, [] { return static_cast<ExecutorBase *>(new IrSequenceRootedExecutor()); });
        R.Register("InsReduceSequenceMesh1DMesh1D", HCCL_CMD_REDUCE, [] { return static_cast<ExecutorBase *>(new IrSequenceRootedExecutor()); });
        R.Register("InsScatterSequenceMesh1DMesh1D", HCCL_CMD_SCATTER, [] { return static_cast<ExecutorBase *>(new IrSequenceRootedExecutor()); });
        R.Register("InsBarrierSequenceMesh1DMesh1D", HCCL_CMD_BARRIER, [] { return static_cast<ExecutorBase *>(new IrSequenceRootedExecutor()); });
        R.Register("InsAllReduceParallelMesh1DMesh1D", HCCL_CMD_ALLREDUCE, [] { return static_cast<ExecutorBase *>(new IrParallelExecutor()); });
        R.Register("InsAllGatherParallelMesh1DMesh1D", HCCL_CMD_ALLGATHER, [] { return static_cast<ExecutorBase *>(new IrParallelExecutor()); });
        R.Register("InsReduceScatterParallelMesh1DMesh1D", HCCL_CMD_REDUCE_SCATTER, [] { return static_cast<ExecutorBase *>(new IrParallelExecutor()); });
        for (const SmAlgoDesc &d : SmAlgorithms())
            R.Register(d.name, d.op, [] { return static_cast<ExecutorBase *>(new SmExecutor()); });
    });
}

}  // namespace hccl
