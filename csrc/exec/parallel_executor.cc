// Parallel executor: AllGather / ReduceScatter / AllReduce on a two-level topology with both levels busy at once.
//
// Every rank's block is cut by the slice planner into (at most) two shares. Share 0 runs its first stage on level 0 (inside
// the server) and its second on level 1 (between servers); share 1 takes the levels in the opposite order. Each share is
// cut into steps, and each share has one queue per level, so that while step i of a share is in its second stage on one
// level, step i + 1 is in its first stage on the other. Queues of one rank hand steps to each other with local notifies;
// every queue has its own bank of notify slots towards the peers, because two queues may talk to the same peer at once.
//
// Stages are the mesh templates of the host-issued engine (InsAllGatherVMesh1D, InsReduceScatterVMesh1D) applied to
// byte ranges of the user buffers, each invocation with a scratch window of its own.
//
// HCCL's counterparts are its Parallel and OmniPipe executors (reference: src/ops/all_reduce/executor/
// ins_v2_all_reduce_parallel_executor.cc:349 runs the intra- and inter-server templates of two data halves at once;
// src/ops/all_gather/executor/ins_v2_all_gather_omnipipe_executor.cc and src/ops/op_common/omnipipe_data_slice_calc.cc
// pipeline per-step slices over two or three axes). Plans with several queues run on the host engine (the copy-engine
// backend takes single-queue plans only).
#include <algorithm>
#include "../common/dtype.h"
#include "../common/log.h"
#include "executor.h"
#include "slice_planner.h"

namespace hccl {
namespace {

constexpr uint32_t kSlotsPerBank = 4;      // the mesh templates use SLOT_ACK .. SLOT_READY
constexpr uint64_t kAlign = 512;

uint64_t Al(uint64_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct Builder {
    const OpParam &p;
    const AlgHierarchyInfo &h;
    Plan *plan;
    uint64_t cclBytes, cclUsed = 0;
    uint32_t es;
    const IrTemplate *ag, *rs;

    uint32_t N(uint32_t level) const { return (uint32_t)h.levelRanks[level].size(); }
    uint32_t Me(uint32_t level) const { return h.myIndex[level]; }
    // first global rank of the server that the level-1 peer k lives in (ranks of a server are consecutive)
    uint32_t Base(uint32_t k) const { return h.levelRanks[1][k] - Me(0); }

    HcclResult Window(uint64_t bytes, uint64_t *off)
    {
        bytes = Al(std::max<uint64_t>(bytes, 1));
        if (cclUsed + bytes > cclBytes) {
            HCCL_ERROR("parallel executor: the schedule needs more than %llu bytes of scratch (raise HCCL_BUFFSIZE)", (unsigned long long)cclBytes);
            return HCCL_E_MEMORY;
        }
        *off = cclUsed;
        cclUsed += bytes;
        return HCCL_SUCCESS;
    }
    TemplateCtx Ctx(uint32_t level) const
    {
        TemplateCtx c;
        c.group = h.levelRanks[level];
        c.me = h.myIndex[level];
        c.elemSize = es;
        return c;
    }
    // appends a template's tasks to `queue`, moving its notify slots into the queue's bank
    HcclResult Run(const IrTemplate *t, const TemplateCtx &c, size_t queue)
    {
        Plan tmp;
        tmp.dtype = plan->dtype;
        tmp.op = plan->op;
        CHK_RET(t->gen(c, &tmp));
        if (tmp.queues.size() > 1) return HCCL_E_INTERNAL;
        plan->EnsureQueues(queue + 1);
        const uint32_t shift = (uint32_t)(queue - 1) * kSlotsPerBank;
        if (!tmp.queues.empty())
            for (Task task : tmp.queues[0]) {
                if (task.type == TaskType::POST || task.type == TaskType::WAIT) {
                    if (task.slot >= kSlotsPerBank) return HCCL_E_INTERNAL;
                    task.slot += shift;
                }
                plan->queues[queue].push_back(task);
            }
        return HCCL_SUCCESS;
    }
    void LocalPost(size_t from, size_t to) { plan->EnsureQueues(std::max(from, to) + 1); plan->queues[from].push_back(Task{TaskType::LOCAL_POST, (uint32_t)to, 0, {}, {}, 0}); }
    void LocalWait(size_t at, size_t from) { plan->EnsureQueues(std::max(from, at) + 1); plan->queues[at].push_back(Task{TaskType::LOCAL_WAIT, (uint32_t)from, 0, {}, {}, 0}); }

    HcclResult AllGatherV(uint32_t level, size_t queue, BufRef in, uint64_t len, const std::vector<uint64_t> &recvOff)
    {
        TemplateCtx c = Ctx(level);
        c.in = in;
        c.out = {BufKind::OUTPUT, 0};
        c.recvBytes.assign(N(level), len);
        c.recvOff = recvOff;
        CHK_RET(Window(len, &c.cclOff));
        c.cclBytes = Al(len);
        return Run(ag, c, queue);
    }
    // Scratch windows are handed out by a bump allocator that has to advance by the same amount on every rank (a template
    // addresses its peers' windows at its own window offset), so the uneven forms take the window size from the caller: the
    // largest slice any rank can hold, not this rank's.
    HcclResult AllGatherVar(uint32_t level, size_t queue, BufRef in, const std::vector<uint64_t> &recvBytes, const std::vector<uint64_t> &recvOff, uint64_t maxSlice)
    {
        TemplateCtx c = Ctx(level);
        c.in = in;
        c.out = {BufKind::OUTPUT, 0};
        c.recvBytes = recvBytes;
        c.recvOff = recvOff;
        CHK_RET(Window(maxSlice, &c.cclOff));
        c.cclBytes = Al(std::max<uint64_t>(maxSlice, 1));
        return Run(ag, c, queue);
    }
    HcclResult ReduceScatterVar(uint32_t level, size_t queue, BufRef in, const std::vector<uint64_t> &sendBytes, const std::vector<uint64_t> &sendOff, BufRef out,
                                uint64_t maxSlice)
    {
        TemplateCtx c = Ctx(level);
        c.in = in;
        c.out = out;
        c.sendBytes = sendBytes;
        c.sendOff = sendOff;
        const uint64_t S = std::max<uint64_t>(Al(maxSlice), kAlign);      // the template spaces its slots by the largest slice it is given, at most this
        CHK_RET(Window(S * N(level), &c.cclOff));
        c.cclBytes = S * N(level);
        return Run(rs, c, queue);
    }

    // ---- one step of a share: byte range [o, o + len) of every rank's block (AllGather / ReduceScatter) or of the vector
    HcclResult AllGatherStep(uint32_t first, size_t q1, size_t q2, uint64_t o, uint64_t len)
    {
        const uint64_t B = (p.blockStride ? p.blockStride : p.count) * es;      // bytes between the per-rank blocks of the user buffers
        const uint32_t n0 = N(0), n1 = N(1), me0 = Me(0);
        const uint32_t myRank = h.levelRanks[0][me0];
        std::vector<uint64_t> off;
        if (first == 1) {
            off.resize(n1);
            for (uint32_t k = 0; k < n1; ++k) off[k] = (uint64_t)h.levelRanks[1][k] * B + o;
            CHK_RET(AllGatherV(1, q1, {BufKind::INPUT, o}, len, off));
            LocalPost(q1, q2);
            LocalWait(q2, q1);
            for (uint32_t s = 0; s < n1; ++s) {                 // forward server s's copy of my column inside my server
                off.resize(n0);
                for (uint32_t j = 0; j < n0; ++j) off[j] = (uint64_t)(Base(s) + j) * B + o;
                CHK_RET(AllGatherV(0, q2, {BufKind::OUTPUT, (uint64_t)h.levelRanks[1][s] * B + o}, len, off));
            }
        } else {
            off.resize(n0);
            for (uint32_t j = 0; j < n0; ++j) off[j] = (uint64_t)h.levelRanks[0][j] * B + o;
            CHK_RET(AllGatherV(0, q1, {BufKind::INPUT, o}, len, off));
            LocalPost(q1, q2);
            LocalWait(q2, q1);
            for (uint32_t j = 0; j < n0; ++j) {                 // forward block j of my server to the other servers
                off.resize(n1);
                for (uint32_t k = 0; k < n1; ++k) off[k] = (uint64_t)(Base(k) + j) * B + o;
                CHK_RET(AllGatherV(1, q2, {BufKind::OUTPUT, (uint64_t)h.levelRanks[0][j] * B + o}, len, off));
            }
        }
        (void)myRank;
        return HCCL_SUCCESS;
    }

    HcclResult ReduceScatterStep(uint32_t first, size_t q1, size_t q2, uint64_t o, uint64_t len)
    {
        const uint64_t B = (p.blockStride ? p.blockStride : p.count) * es;      // bytes between the per-rank blocks of the user buffers
        const uint32_t n0 = N(0), n1 = N(1);
        const uint32_t second = 1 - first, nf = N(first), ns = N(second);
        // first stage: one reduce-scatter per member of the OTHER level's group, each leaving a partial sum in the work area
        uint64_t work;
        CHK_RET(Window(Al(len) * ns, &work));
        for (uint32_t m = 0; m < ns; ++m) {
            std::vector<uint64_t> sb(nf, len), so(nf);
            for (uint32_t x = 0; x < nf; ++x) {
                // block of the rank at (level-0 position, server): first = 0 walks my server's... positions j of server m; first = 1 walks servers k at position m
                const uint32_t rank = first == 0 ? Base(m) + x : Base(x) + m;
                so[x] = (uint64_t)rank * B + o;
            }
            CHK_RET(ReduceScatterVar(first, q1, {BufKind::INPUT, 0}, sb, so, {BufKind::CCL, work + (uint64_t)m * Al(len)}, len));
        }
        LocalPost(q1, q2);
        LocalWait(q2, q1);
        std::vector<uint64_t> sb(ns, len), so(ns);
        for (uint32_t m = 0; m < ns; ++m) so[m] = (uint64_t)m * Al(len);
        (void)n0; (void)n1;
        return ReduceScatterVar(second, q2, {BufKind::CCL, work}, sb, so, {BufKind::OUTPUT, o}, len);
    }

    // element slices of [o, o + len) over n ranks, in bytes
    void Cut(uint64_t len, uint32_t n, std::vector<uint64_t> *lens, std::vector<uint64_t> *offs) const
    {
        const uint64_t cnt = len / es, per = (cnt + n - 1) / n;
        lens->resize(n);
        offs->resize(n);
        for (uint32_t j = 0; j < n; ++j) {
            const uint64_t lo = std::min(cnt, per * j), hi = std::min(cnt, per * (j + 1));
            (*offs)[j] = lo * es;
            (*lens)[j] = (hi - lo) * es;
        }
    }
    // AllReduce of the sub-vector [o, o + len): reduce-scatter on `first` (queue q1), reduce-scatter + all-gather of my slice on
    // the other level (queue q2), all-gather on `first` (queue q1, after every step's reduce-scatter)
    HcclResult AllReduceDown(uint32_t first, size_t q1, size_t q2, uint64_t o, uint64_t len)
    {
        const uint32_t second = 1 - first;
        std::vector<uint64_t> la, oa, lb, ob;
        Cut(len, N(first), &la, &oa);
        std::vector<uint64_t> so(oa);
        for (auto &v : so) v += o;
        const uint64_t mine = o + oa[Me(first)], mineLen = la[Me(first)];
        CHK_RET(ReduceScatterVar(first, q1, {BufKind::INPUT, 0}, la, so, {BufKind::OUTPUT, mine}, la[0]));
        LocalPost(q1, q2);
        LocalWait(q2, q1);
        Cut(mineLen, N(second), &lb, &ob);
        std::vector<uint64_t> lmax, omax;
        Cut(la[0], N(second), &lmax, &omax);                       // la[0] is the longest first-level slice, lmax[0] the longest second-level one
        std::vector<uint64_t> so2(ob), ro2(ob);
        for (auto &v : so2) v += mine;
        for (auto &v : ro2) v += mine;
        CHK_RET(ReduceScatterVar(second, q2, {BufKind::OUTPUT, 0}, lb, so2, {BufKind::OUTPUT, mine + ob[Me(second)]}, lmax[0]));
        CHK_RET(AllGatherVar(second, q2, {BufKind::OUTPUT, mine + ob[Me(second)]}, lb, ro2, lmax[0]));
        LocalPost(q2, q1);
        return HCCL_SUCCESS;
    }
    HcclResult AllReduceUp(uint32_t first, size_t q1, size_t q2, uint64_t o, uint64_t len)
    {
        std::vector<uint64_t> la, oa;
        Cut(len, N(first), &la, &oa);
        std::vector<uint64_t> ro(oa);
        for (auto &v : ro) v += o;
        LocalWait(q1, q2);
        return AllGatherVar(first, q1, {BufKind::OUTPUT, o + oa[Me(first)]}, la, ro, la[0]);
    }
};

}  // namespace

HcclResult GenParallelPlan(const OpParam &p, const TopoInfo &topo, uint64_t cclBytes, Plan *plan, SlicePlan *slicesOut)
{
    AlgHierarchyInfo h;
    CHK_RET(TopoMatch(topo, TopoMatchKind::TWO_LEVEL, &h));       // super-pods fold into the upper level
    if (h.levelRanks.size() != 2) return HCCL_E_NOT_SUPPORT;
    const uint32_t n0 = (uint32_t)h.levelRanks[0].size(), n1 = (uint32_t)h.levelRanks[1].size();
    for (uint32_t j = 0; j < n0; ++j)
        if (h.levelRanks[0][j] != h.levelRanks[0][0] + j) return HCCL_E_NOT_SUPPORT;        // ranks of a server are consecutive
    for (uint32_t k = 0; k < n1; ++k)
        if (h.levelRanks[1][k] < h.myIndex[0]) return HCCL_E_NOT_SUPPORT;
    PipeOp op;
    switch (p.opType) {
        case HCCL_CMD_ALLGATHER: op = PipeOp::ALLGATHER; break;
        case HCCL_CMD_REDUCE_SCATTER: op = PipeOp::REDUCE_SCATTER; break;
        case HCCL_CMD_ALLREDUCE: op = PipeOp::ALLREDUCE; break;
        default: return HCCL_E_NOT_SUPPORT;
    }
    RegisterBuiltinIrTemplates();
    const uint32_t es = DataTypeSize(p.dtype);
    Builder b{p, h, plan, cclBytes, 0, es, IrTemplateRegistry::Instance().Find("InsAllGatherVMesh1D"), IrTemplateRegistry::Instance().Find("InsReduceScatterVMesh1D")};
    if (!b.ag || !b.rs || es == 0) return HCCL_E_INTERNAL;
    plan->dtype = p.dtype;
    plan->op = p.reduceOp;
    plan->EnsureQueues(1);

    AxisSpec a0{n0, topo.levelBandwidth.size() > 0 ? topo.levelBandwidth[0] : 770.0, 2.0};
    AxisSpec a1{n1, FoldedUpperBandwidth(topo, 50.0), 5.0};
    SlicePlan sp;
    CHK_RET(PlanSlices(op, a0, a1, p.count * es, kAlign, 4, &sp));
    if (slicesOut) *slicesOut = sp;
    // queues: 0 = the caller's (empty here: the engine joins all queues of a plan), then two per share
    for (size_t si = 0; si < sp.shares.size(); ++si) {
        const PipeShare &s = sp.shares[si];
        const size_t q1 = 1 + 2 * si, q2 = 2 + 2 * si;
        plan->EnsureQueues(q2 + 1);
        for (uint32_t i = 0; i < s.steps; ++i) {
            uint64_t o, len;
            StepRange(s, kAlign, i, &o, &len);
            if (len == 0) continue;
            if (op == PipeOp::ALLGATHER) CHK_RET(b.AllGatherStep(s.firstLevel, q1, q2, o, len));
            else if (op == PipeOp::REDUCE_SCATTER) CHK_RET(b.ReduceScatterStep(s.firstLevel, q1, q2, o, len));
            else CHK_RET(b.AllReduceDown(s.firstLevel, q1, q2, o, len));
        }
        if (op == PipeOp::ALLREDUCE)
            for (uint32_t i = 0; i < s.steps; ++i) {
                uint64_t o, len;
                StepRange(s, kAlign, i, &o, &len);
                if (len == 0) continue;
                CHK_RET(b.AllReduceUp(s.firstLevel, q1, q2, o, len));
            }
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
