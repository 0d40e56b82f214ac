#include "ir_templates.h"
#include <algorithm>
#include <mutex>
#include "../common/log.h"
#include "../topo/topo_info.h"

namespace hccl {

IrTemplateRegistry &IrTemplateRegistry::Instance()
{
    static IrTemplateRegistry r;
    return r;
}
void IrTemplateRegistry::Register(const IrTemplate &t) { map_[t.name] = t; }
const IrTemplate *IrTemplateRegistry::Find(const std::string &name) const
{
    auto it = map_.find(name);
    return it == map_.end() ? nullptr : &it->second;
}
std::vector<std::string> IrTemplateRegistry::Names(HcclCMDType op) const
{
    std::vector<std::string> v;
    for (auto &kv : map_) if (kv.second.op == op) v.push_back(kv.first);
    return v;
}

namespace {

constexpr uint64_t kAlign = 512;
uint64_t AlignUp(uint64_t v, uint64_t a = kAlign) { return (v + a - 1) / a * a; }

// Emission helper bound to one queue of the plan.
struct Emit {
    const TemplateCtx &c;
    Plan *p;
    size_t qi;
    Emit(const TemplateCtx &ctx, Plan *plan, size_t queue = 0) : c(ctx), p(plan), qi(queue) { p->EnsureQueues(queue + 1); }
    std::vector<Task> &q() { return p->queues[qi]; }
    BufRef Ccl(uint64_t off) const { return BufRef{BufKind::CCL, c.cclOff + off}; }
    static BufRef At(BufRef b, uint64_t off) { b.off += off; return b; }
    void Copy(BufRef d, BufRef s, uint64_t n) { if (n) q().push_back(Task{TaskType::LOCAL_COPY, 0, 0, d, s, n}); }
    void Reduce(BufRef d, BufRef s, uint64_t n) { if (n) q().push_back(Task{TaskType::LOCAL_REDUCE, 0, 0, d, s, n}); }
    void Write(uint32_t peerIdx, BufRef remote, BufRef s, uint64_t n) { if (n) q().push_back(Task{TaskType::WRITE, c.group[peerIdx], 0, remote, s, n}); }
    void Read(uint32_t peerIdx, BufRef d, BufRef remote, uint64_t n) { if (n) q().push_back(Task{TaskType::READ, c.group[peerIdx], 0, d, remote, n}); }
    void Post(uint32_t peerIdx, uint32_t slot) { q().push_back(Task{TaskType::POST, c.group[peerIdx], slot, {}, {}, 0}); }
    void Wait(uint32_t peerIdx, uint32_t slot) { q().push_back(Task{TaskType::WAIT, c.group[peerIdx], slot, {}, {}, 0}); }
    void PostAll(uint32_t slot) { for (uint32_t k = 1; k < c.N(); ++k) Post((c.me + k) % c.N(), slot); }
    void WaitAll(uint32_t slot) { for (uint32_t k = 1; k < c.N(); ++k) Wait((c.me + k) % c.N(), slot); }
    void Barrier(uint32_t slot) { PostAll(slot); WaitAll(slot); }
};

// Element slices of `count` over n ranks: the first (count % n) slices carry one extra element.
struct Slices {
    uint64_t base, rem, es;
    Slices(uint64_t count, uint32_t n, uint32_t elemSize) : base(count / n), rem(count % n), es(elemSize) {}
    uint64_t Len(uint32_t j) const { return (base + (j < rem ? 1 : 0)) * es; }
    uint64_t Off(uint32_t j) const { return (base * j + std::min<uint64_t>(j, rem)) * es; }
    uint64_t MaxLen() const { return AlignUp((base + (rem ? 1 : 0)) * es); }
};

uint32_t Mod(int64_t v, uint32_t n) { int64_t m = v % (int64_t)n; return (uint32_t)(m < 0 ? m + n : m); }

uint32_t NhrStepCount(uint32_t n)
{
    uint32_t s = 0;
    for (uint32_t t = n - 1; t != 0; t >>= 1) ++s;
    return s;
}
// staging slices needed over all steps of one NHR phase
uint64_t NhrStageSlices(uint32_t n)
{
    uint64_t tot = 0;
    for (uint32_t s = 0; s < NhrStepCount(n); ++s) tot += (n - 1 + (1u << s)) / (2u << s);
    return tot;
}

// ---- reduce-scatter / all-gather phases over per-rank blocks located at work(j), shared by several templates
using BlockRef = std::function<BufRef(uint32_t)>;
using BlockLen = std::function<uint64_t(uint32_t)>;

void NhrReduceScatterPhase(Emit &e, const BlockRef &work, const BlockLen &len, uint64_t stageOff, uint64_t maxLen)
{
    uint32_t n = e.c.N(), me = e.c.me;
    uint64_t off = stageOff;
    uint32_t nSteps = NhrStepCount(n);
    for (uint32_t s = 0; s < nSteps; ++s) {
        uint32_t delta = 1u << s, stride = delta << 1, nSl = (n - 1 + delta) / stride;
        uint32_t sendTo = Mod((int64_t)me - delta, n), recvFrom = (me + delta) % n;
        for (uint32_t k = 0; k < nSl; ++k) {
            uint32_t tx = Mod((int64_t)sendTo - (int64_t)k * stride, n);
            e.Write(sendTo, e.Ccl(off + k * maxLen), work(tx), len(tx));
        }
        e.Post(sendTo, SLOT_STEP_BASE + s);
        e.Wait(recvFrom, SLOT_STEP_BASE + s);
        for (uint32_t k = 0; k < nSl; ++k) {
            uint32_t rx = Mod((int64_t)me - (int64_t)k * stride, n);
            e.Reduce(work(rx), e.Ccl(off + k * maxLen), len(rx));
        }
        off += (uint64_t)nSl * maxLen;
    }
}

void NhrAllGatherPhase(Emit &e, const BlockRef &work, const BlockLen &len, uint64_t stageOff, uint64_t maxLen)
{
    uint32_t n = e.c.N(), me = e.c.me;
    uint64_t off = stageOff;
    uint32_t nSteps = NhrStepCount(n);
    for (uint32_t t = 0; t < nSteps; ++t) {
        uint32_t delta = 1u << (nSteps - 1 - t), stride = delta << 1, nSl = (n - 1 + delta) / stride;
        uint32_t sendTo = (me + delta) % n, recvFrom = Mod((int64_t)me - delta, n);
        for (uint32_t k = 0; k < nSl; ++k) {
            uint32_t tx = Mod((int64_t)me - (int64_t)k * stride, n);
            e.Write(sendTo, e.Ccl(off + k * maxLen), work(tx), len(tx));
        }
        e.Post(sendTo, SLOT_STEP_BASE + 8 + t);
        e.Wait(recvFrom, SLOT_STEP_BASE + 8 + t);
        for (uint32_t k = 0; k < nSl; ++k) {
            uint32_t rx = Mod((int64_t)me - delta - (int64_t)k * stride, n);
            e.Copy(work(rx), e.Ccl(off + k * maxLen), len(rx));
        }
        off += (uint64_t)nSl * maxLen;
    }
}

uint64_t Unlimited(uint32_t, uint32_t, uint64_t) { return 0; }

// ================================================================================================ AllReduce
HcclResult GenAllReduceOneShot(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Write(peer, e.Ccl(c.me * S), c.in, B);
        e.Post(peer, SLOT_DATA);
    }
    e.Copy(e.Ccl(c.me * S), c.in, B);
    e.WaitAll(SLOT_DATA);
    e.Copy(c.out, e.Ccl(0), B);
    for (uint32_t r = 1; r < n; ++r) e.Reduce(c.out, e.Ccl(r * S), B);   // rank order on every rank: bit-identical results
    return HCCL_SUCCESS;
}

HcclResult GenAllReduceTwoShot(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    Slices sl(c.count, n, c.elemSize);
    uint64_t M = sl.MaxLen();
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Write(peer, e.Ccl(c.me * M), Emit::At(c.in, sl.Off(peer)), sl.Len(peer));
        e.Post(peer, SLOT_DATA);
    }
    e.Copy(e.Ccl(c.me * M), Emit::At(c.in, sl.Off(c.me)), sl.Len(c.me));
    e.WaitAll(SLOT_DATA);
    BufRef res = e.Ccl((uint64_t)n * M);
    e.Copy(res, e.Ccl(0), sl.Len(c.me));
    for (uint32_t r = 1; r < n; ++r) e.Reduce(res, e.Ccl(r * M), sl.Len(c.me));
    e.Copy(Emit::At(c.out, sl.Off(c.me)), res, sl.Len(c.me));
    e.Barrier(SLOT_READY);
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Read(peer, Emit::At(c.out, sl.Off(peer)), e.Ccl((uint64_t)n * M), sl.Len(peer));
    }
    return HCCL_SUCCESS;
}

HcclResult GenAllReduceRing(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N(), me = c.me;
    Slices sl(c.count, n, c.elemSize);
    uint64_t M = sl.MaxLen();
    if (!c.inPlace) e.Copy(c.out, c.in, c.count * c.elemSize);
    uint32_t next = (me + 1) % n, prev = Mod((int64_t)me - 1, n);
    for (uint32_t s = 0; s + 1 < n; ++s) {
        uint32_t tx = Mod((int64_t)me - s, n), rx = Mod((int64_t)me - s - 1, n);
        e.Write(next, e.Ccl(s * M), Emit::At(c.out, sl.Off(tx)), sl.Len(tx));
        e.Post(next, SLOT_DATA);
        e.Wait(prev, SLOT_DATA);
        e.Reduce(Emit::At(c.out, sl.Off(rx)), e.Ccl(s * M), sl.Len(rx));
    }
    for (uint32_t s = 0; s + 1 < n; ++s) {
        uint32_t tx = Mod((int64_t)me + 1 - s, n), rx = Mod((int64_t)me - s, n);
        e.Write(next, e.Ccl((n - 1 + s) * M), Emit::At(c.out, sl.Off(tx)), sl.Len(tx));
        e.Post(next, SLOT_DATA);
        e.Wait(prev, SLOT_DATA);
        e.Copy(Emit::At(c.out, sl.Off(rx)), e.Ccl((n - 1 + s) * M), sl.Len(rx));
    }
    return HCCL_SUCCESS;
}

HcclResult GenAllReduceNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    Slices sl(c.count, n, c.elemSize);
    uint64_t M = sl.MaxLen();
    if (!c.inPlace) e.Copy(c.out, c.in, c.count * c.elemSize);
    BlockRef work = [&](uint32_t j) { return Emit::At(c.out, sl.Off(j)); };
    BlockLen len = [&](uint32_t j) { return sl.Len(j); };
    NhrReduceScatterPhase(e, work, len, 0, M);
    NhrAllGatherPhase(e, work, len, NhrStageSlices(n) * M, M);
    return HCCL_SUCCESS;
}

// ================================================================================================ AllGather
HcclResult GenAllGatherMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    uint64_t B = c.count * c.elemSize;
    e.Copy(e.Ccl(0), c.in, B);
    e.Barrier(SLOT_READY);
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Read(peer, Emit::At(c.out, peer * c.outStride), e.Ccl(0), B);
    }
    if (!c.inPlace) e.Copy(Emit::At(c.out, c.me * c.outStride), c.in, B);
    return HCCL_SUCCESS;
}

HcclResult GenAllGatherRing(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N(), me = c.me;
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    if (!c.inPlace) e.Copy(Emit::At(c.out, me * c.outStride), c.in, B);
    uint32_t next = (me + 1) % n, prev = Mod((int64_t)me - 1, n);
    for (uint32_t s = 0; s + 1 < n; ++s) {
        uint32_t tx = Mod((int64_t)me - s, n), rx = Mod((int64_t)me - s - 1, n);
        e.Write(next, e.Ccl(s * S), Emit::At(c.out, tx * c.outStride), B);
        e.Post(next, SLOT_DATA);
        e.Wait(prev, SLOT_DATA);
        e.Copy(Emit::At(c.out, rx * c.outStride), e.Ccl(s * S), B);
    }
    return HCCL_SUCCESS;
}

HcclResult GenAllGatherNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    if (!c.inPlace) e.Copy(Emit::At(c.out, c.me * c.outStride), c.in, B);
    BlockRef work = [&](uint32_t j) { return Emit::At(c.out, j * c.outStride); };
    BlockLen len = [&](uint32_t) { return B; };
    NhrAllGatherPhase(e, work, len, 0, S);
    return HCCL_SUCCESS;
}

// ================================================================================================ ReduceScatter
HcclResult GenReduceScatterMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Write(peer, e.Ccl(c.me * S), Emit::At(c.in, peer * c.inStride), B);
        e.Post(peer, SLOT_DATA);
    }
    e.Copy(e.Ccl(c.me * S), Emit::At(c.in, c.me * c.inStride), B);
    e.WaitAll(SLOT_DATA);
    e.Copy(c.out, e.Ccl(0), B);
    for (uint32_t r = 1; r < n; ++r) e.Reduce(c.out, e.Ccl(r * S), B);
    return HCCL_SUCCESS;
}

HcclResult GenReduceScatterRing(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N(), me = c.me;
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    if (n == 1) { e.Copy(c.out, c.in, B); return HCCL_SUCCESS; }
    uint32_t next = (me + 1) % n, prev = Mod((int64_t)me - 1, n);
    for (uint32_t s = 0; s + 1 < n; ++s) {
        uint32_t tx = Mod((int64_t)me - 1 - s, n), rx = Mod((int64_t)me - 2 - s, n);
        BufRef src = s == 0 ? Emit::At(c.in, tx * c.inStride) : e.Ccl((s - 1) * S);
        e.Write(next, e.Ccl(s * S), src, B);
        e.Post(next, SLOT_DATA);
        e.Wait(prev, SLOT_DATA);
        e.Reduce(e.Ccl(s * S), Emit::At(c.in, rx * c.inStride), B);   // staged partial += my contribution
    }
    e.Copy(c.out, e.Ccl((n - 2) * S), B);
    return HCCL_SUCCESS;
}

HcclResult GenReduceScatterNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    for (uint32_t j = 0; j < n; ++j) e.Copy(e.Ccl(j * S), Emit::At(c.in, j * c.inStride), B);   // private working copy
    BlockRef work = [&](uint32_t j) { return e.Ccl(j * S); };
    BlockLen len = [&](uint32_t) { return B; };
    NhrReduceScatterPhase(e, work, len, (uint64_t)n * S, S);
    e.Copy(c.out, e.Ccl(c.me * S), B);
    return HCCL_SUCCESS;
}

// ================================================================================================ Broadcast
HcclResult GenBroadcastOneShot(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint64_t B = c.count * c.elemSize;
    if (c.me == c.root) {
        e.Copy(e.Ccl(0), c.out, B);
        e.PostAll(SLOT_READY);
    } else {
        e.Wait(c.root, SLOT_READY);
        e.Read(c.root, c.out, e.Ccl(0), B);
    }
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

HcclResult GenBroadcastTwoShot(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    Slices sl(c.count, n, c.elemSize);
    if (c.me == c.root) {
        for (uint32_t k = 1; k < n; ++k) {
            uint32_t peer = (c.me + k) % n;
            e.Write(peer, e.Ccl(sl.Off(peer)), Emit::At(c.out, sl.Off(peer)), sl.Len(peer));
            e.Post(peer, SLOT_DATA);
        }
        e.Copy(e.Ccl(sl.Off(c.me)), Emit::At(c.out, sl.Off(c.me)), sl.Len(c.me));
    } else {
        e.Wait(c.root, SLOT_DATA);
    }
    e.Barrier(SLOT_READY);
    if (c.me != c.root) {
        for (uint32_t k = 1; k < n; ++k) {
            uint32_t peer = (c.me + k) % n;
            e.Read(peer, Emit::At(c.out, sl.Off(peer)), e.Ccl(sl.Off(peer)), sl.Len(peer));
        }
        e.Copy(Emit::At(c.out, sl.Off(c.me)), e.Ccl(sl.Off(c.me)), sl.Len(c.me));
    }
    e.Barrier(SLOT_FIN);   // nobody leaves while a peer may still read its slice
    return HCCL_SUCCESS;
}

// ================================================================================================ Reduce / Scatter
HcclResult GenReduceMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    if (c.me != c.root) {
        e.Write(c.root, e.Ccl(c.me * S), c.in, B);
        e.Post(c.root, SLOT_DATA);
    } else {
        e.Copy(e.Ccl(c.me * S), c.in, B);
        e.WaitAll(SLOT_DATA);
        e.Copy(c.out, e.Ccl(0), B);
        for (uint32_t r = 1; r < n; ++r) e.Reduce(c.out, e.Ccl(r * S), B);
    }
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// Two-shot reduce: mesh reduce-scatter, then the owners write their reduced slices to the root.
HcclResult GenReduceTwoShot(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    Slices sl(c.count, n, c.elemSize);
    uint64_t M = sl.MaxLen();
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Write(peer, e.Ccl(c.me * M), Emit::At(c.in, sl.Off(peer)), sl.Len(peer));
        e.Post(peer, SLOT_DATA);
    }
    e.Copy(e.Ccl(c.me * M), Emit::At(c.in, sl.Off(c.me)), sl.Len(c.me));
    e.WaitAll(SLOT_DATA);
    BufRef res = e.Ccl((uint64_t)n * M);
    e.Copy(res, e.Ccl(0), sl.Len(c.me));
    for (uint32_t r = 1; r < n; ++r) e.Reduce(res, e.Ccl(r * M), sl.Len(c.me));
    if (c.me != c.root) {
        e.Write(c.root, e.Ccl((uint64_t)(n + 1 + c.me) * M), res, sl.Len(c.me));
        e.Post(c.root, SLOT_READY);
    } else {
        e.Copy(Emit::At(c.out, sl.Off(c.me)), res, sl.Len(c.me));
        for (uint32_t k = 1; k < n; ++k) {
            uint32_t peer = (c.me + k) % n;
            e.Wait(peer, SLOT_READY);
            e.Copy(Emit::At(c.out, sl.Off(peer)), e.Ccl((uint64_t)(n + 1 + peer) * M), sl.Len(peer));
        }
    }
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// With sendBytes / sendOff set the blocks have their own lengths and offsets in the root's buffer (the multi-level executors scatter
// the uneven slices of a vector this way); inPlace then says that the root's own block already sits where it belongs.
HcclResult GenScatterMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    const bool v = !c.sendBytes.empty();
    if (v && (c.sendBytes.size() != n || c.sendOff.size() != n)) return HCCL_E_INTERNAL;
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    if (v) { S = 0; for (uint64_t b : c.sendBytes) S = std::max(S, AlignUp(b)); }
    auto len = [&](uint32_t j) { return v ? c.sendBytes[j] : B; };
    auto off = [&](uint32_t j) { return v ? c.sendOff[j] : (uint64_t)j * c.inStride; };
    if (c.me == c.root) {
        for (uint32_t j = 0; j < n; ++j) if (j != c.me) e.Copy(e.Ccl(j * S), Emit::At(c.in, off(j)), len(j));
        e.PostAll(SLOT_READY);
        if (!(v && c.inPlace)) e.Copy(c.out, Emit::At(c.in, off(c.me)), len(c.me));
    } else {
        e.Wait(c.root, SLOT_READY);
        e.Read(c.root, c.out, e.Ccl(c.me * S), len(c.me));
    }
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// Gather of blocks of their own lengths at the root (recvBytes / recvOff: block j's length and its offset in the root's buffer); a
// building block of the multi-level Reduce (reference: src/ops/reduce/template/aicpu/ins_temp_gather_mesh_1D_intra.cc).
HcclResult GenGatherMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    if (c.recvBytes.size() != n || c.recvOff.size() != n) return HCCL_E_INTERNAL;
    if (c.me != c.root) {
        e.Copy(e.Ccl(0), c.in, c.recvBytes[c.me]);
        e.Post(c.root, SLOT_READY);
    } else {
        e.Copy(Emit::At(c.out, c.recvOff[c.me]), c.in, c.recvBytes[c.me]);
        for (uint32_t k = 1; k < n; ++k) {
            uint32_t peer = (c.me + k) % n;
            e.Wait(peer, SLOT_READY);
            e.Read(peer, Emit::At(c.out, c.recvOff[peer]), e.Ccl(0), c.recvBytes[peer]);
        }
    }
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// Tree scatter ("NHR" in HCCL's scatter family, reference: src/ops/scatter/template/aicpu/ins_temp_scatter_nhr.cc): ranks are numbered
// relative to the root; in the step of distance d (d = P/2, P/4, ..., 1 with P the power of two at or above n) every rank whose
// relative number is a multiple of 2d hands the blocks of the d ranks that follow its own d to the rank at distance d. The root sends
// from the user buffer, everyone else from the scratch it received into (its own block first), so a block crosses ceil(log2 n) links
// at most and the root sends n - 1 blocks in ceil(log2 n) messages instead of n - 1.
HcclResult GenScatterNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    const uint32_t n = c.N(), r = Mod((int64_t)c.me - c.root, n);
    const uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    auto abs = [&](uint32_t rel) { return (rel + c.root) % n; };
    uint32_t P = 1;
    while (P < n) P <<= 1;
    uint32_t step = 0;
    for (uint32_t d = P >> 1; d >= 1; d >>= 1, ++step) {
        if (r % (2 * d) == 0 && r + d < n) {
            const uint32_t to = r + d, hi = std::min(r + 2 * d, n);
            for (uint32_t q = to; q < hi; ++q) {
                BufRef src = r == 0 ? Emit::At(c.in, (uint64_t)abs(q) * c.inStride) : e.Ccl((uint64_t)(q - r) * S);
                e.Write(abs(to), e.Ccl((uint64_t)(q - to) * S), src, B);
            }
            e.Post(abs(to), SLOT_STEP_BASE + step);
        } else if (r % (2 * d) == d) {
            e.Wait(abs(r - d), SLOT_STEP_BASE + step);
        }
    }
    if (r == 0) e.Copy(c.out, Emit::At(c.in, (uint64_t)c.me * c.inStride), B);
    else e.Copy(c.out, e.Ccl(0), B);
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// Broadcast as a scatter of slices from the root followed by the NHR all-gather (reference: src/ops/broadcast/template/aicpu/
// ins_temp_broadcast_nhr.cc): every rank forwards what it has in ceil(log2 n) steps, so the root sends the payload once.
HcclResult GenBroadcastNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    const uint32_t n = c.N();
    Slices sl(c.count, n, c.elemSize);
    const uint64_t M = sl.MaxLen();
    if (c.me == c.root) {
        for (uint32_t k = 1; k < n; ++k) {
            uint32_t peer = (c.me + k) % n;
            e.Write(peer, e.Ccl(0), Emit::At(c.out, sl.Off(peer)), sl.Len(peer));
            e.Post(peer, SLOT_DATA);
        }
    } else {
        e.Wait(c.root, SLOT_DATA);
        e.Copy(Emit::At(c.out, sl.Off(c.me)), e.Ccl(0), sl.Len(c.me));
    }
    BlockRef work = [&](uint32_t j) { return Emit::At(c.out, sl.Off(j)); };
    BlockLen len = [&](uint32_t j) { return sl.Len(j); };
    NhrAllGatherPhase(e, work, len, M, M);
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// Reduce as the NHR reduce-scatter on a private copy of the input followed by a gather of the reduced slices at the root
// (reference: src/ops/reduce/template/aicpu/reduce_nhr.cc).
HcclResult GenReduceNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    const uint32_t n = c.N();
    Slices sl(c.count, n, c.elemSize);
    const uint64_t M = sl.MaxLen(), stage = NhrStageSlices(n);
    for (uint32_t j = 0; j < n; ++j) e.Copy(e.Ccl(j * M), Emit::At(c.in, sl.Off(j)), sl.Len(j));
    BlockRef work = [&](uint32_t j) { return e.Ccl(j * M); };
    BlockLen len = [&](uint32_t j) { return sl.Len(j); };
    NhrReduceScatterPhase(e, work, len, (uint64_t)n * M, M);
    const uint64_t gather = ((uint64_t)n + stage) * M;
    if (c.me != c.root) {
        e.Write(c.root, e.Ccl(gather + c.me * M), e.Ccl(c.me * M), sl.Len(c.me));
        e.Post(c.root, SLOT_READY);
    } else {
        e.Copy(Emit::At(c.out, sl.Off(c.me)), e.Ccl(c.me * M), sl.Len(c.me));
        for (uint32_t k = 1; k < n; ++k) {
            uint32_t peer = (c.me + k) % n;
            e.Wait(peer, SLOT_READY);
            e.Copy(Emit::At(c.out, sl.Off(peer)), e.Ccl(gather + peer * M), sl.Len(peer));
        }
    }
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// ================================================================================================ AlltoAll family
HcclResult GenAlltoAllMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    uint64_t B = c.count * c.elemSize, S = AlignUp(B);
    for (uint32_t j = 0; j < n; ++j) if (j != c.me) e.Copy(e.Ccl(j * S), Emit::At(c.in, j * c.inStride), B);
    e.Barrier(SLOT_READY);
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Read(peer, Emit::At(c.out, peer * c.outStride), e.Ccl(c.me * S), B);
    }
    e.Copy(Emit::At(c.out, c.me * c.outStride), Emit::At(c.in, c.me * c.inStride), B);
    return HCCL_SUCCESS;
}

// Pairwise regions with credit: the sender owns region [me] of the receiver's scratch, refilled round by round
// under an ACK/DATA handshake (HCCL's AlltoAllV kernels chunk-loop with credit + data flags the same way;
// reference: src/ops/all_to_all_v/template/aiv/kernel/aiv_all_to_all_v_mesh_1D.h:164-240).
HcclResult GenAlltoAllVMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    if (c.sendBytes.size() != n || c.recvBytes.size() != n || c.sendOff.size() != n || c.recvOff.size() != n) return HCCL_E_INTERNAL;
    uint64_t region = c.cclBytes / n / kAlign * kAlign;
    if (region == 0) return HCCL_E_MEMORY;
    auto rounds = [&](uint64_t b) { return (b + region - 1) / region; };
    uint64_t R = 0;
    for (uint32_t j = 0; j < n; ++j) if (j != c.me) R = std::max({R, rounds(c.sendBytes[j]), rounds(c.recvBytes[j])});
    for (uint64_t k = 0; k < R; ++k) {
        for (uint32_t d = 1; d < n; ++d) {
            uint32_t peer = (c.me + d) % n;
            if (k >= rounds(c.sendBytes[peer])) continue;
            if (k > 0) e.Wait(peer, SLOT_ACK);
            uint64_t len = std::min(region, c.sendBytes[peer] - k * region);
            e.Write(peer, e.Ccl(c.me * region), Emit::At(c.in, c.sendOff[peer] + k * region), len);
            e.Post(peer, SLOT_DATA);
        }
        for (uint32_t d = 1; d < n; ++d) {
            uint32_t peer = Mod((int64_t)c.me - d, n);
            if (k >= rounds(c.recvBytes[peer])) continue;
            e.Wait(peer, SLOT_DATA);
            uint64_t len = std::min(region, c.recvBytes[peer] - k * region);
            e.Copy(Emit::At(c.out, c.recvOff[peer] + k * region), e.Ccl(peer * region), len);
            if (k + 1 < rounds(c.recvBytes[peer])) e.Post(peer, SLOT_ACK);
        }
    }
    e.Copy(Emit::At(c.out, c.recvOff[c.me]), Emit::At(c.in, c.sendOff[c.me]), c.sendBytes[c.me]);
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

HcclResult GenAllGatherVMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    if (c.recvBytes.size() != n || c.recvOff.size() != n) return HCCL_E_INTERNAL;
    e.Copy(e.Ccl(0), c.in, c.recvBytes[c.me]);
    e.Barrier(SLOT_READY);
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Read(peer, Emit::At(c.out, c.recvOff[peer]), e.Ccl(0), c.recvBytes[peer]);
    }
    e.Copy(Emit::At(c.out, c.recvOff[c.me]), c.in, c.recvBytes[c.me]);
    return HCCL_SUCCESS;
}

HcclResult GenReduceScatterVMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    if (c.sendBytes.size() != n || c.sendOff.size() != n) return HCCL_E_INTERNAL;
    uint64_t S = 0;
    for (uint64_t b : c.sendBytes) S = std::max(S, AlignUp(b));
    for (uint32_t k = 1; k < n; ++k) {
        uint32_t peer = (c.me + k) % n;
        e.Write(peer, e.Ccl(c.me * S), Emit::At(c.in, c.sendOff[peer]), c.sendBytes[peer]);
        e.Post(peer, SLOT_DATA);
    }
    uint64_t mine = c.sendBytes[c.me];
    e.Copy(e.Ccl(c.me * S), Emit::At(c.in, c.sendOff[c.me]), mine);
    e.WaitAll(SLOT_DATA);
    e.Copy(c.out, e.Ccl(0), mine);
    for (uint32_t r = 1; r < n; ++r) e.Reduce(c.out, e.Ccl(r * S), mine);
    return HCCL_SUCCESS;
}

// ================================================================================================ Barrier
HcclResult GenBarrierMesh(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    e.Barrier(SLOT_FIN);
    return HCCL_SUCCESS;
}

// Dissemination barrier: ceil(log2 n) rounds (the latency-optimal form HCCL uses as "NHR" barrier).
HcclResult GenBarrierNhr(const TemplateCtx &c, Plan *p)
{
    Emit e(c, p);
    uint32_t n = c.N();
    for (uint32_t s = 0, d = 1; d < n; ++s, d <<= 1) {
        e.Post((c.me + d) % n, SLOT_STEP_BASE + s);
        e.Wait(Mod((int64_t)c.me - d, n), SLOT_STEP_BASE + s);
    }
    return HCCL_SUCCESS;
}

uint64_t PerN(uint32_t n, uint32_t es, uint64_t ccl, double mult)
{
    // elements such that mult * count * es (+ alignment slack) fits
    if (ccl <= (uint64_t)(n + 2) * 2 * kAlign) return 0;
    uint64_t usable = ccl - (uint64_t)(n + 2) * 2 * kAlign;
    uint64_t c = (uint64_t)((double)usable / mult) / es;
    c -= c % 128;
    return std::max<uint64_t>(c, 128);
}

std::once_flag g_once;

}  // namespace

void RegisterBuiltinIrTemplates()
{
    std::call_once(g_once, [] {
        auto &R = IrTemplateRegistry::Instance();
        auto reg = [&](const char *name, HcclCMDType op, std::function<HcclResult(const TemplateCtx &, Plan *)> gen,
                       std::function<uint64_t(uint32_t, uint32_t, uint64_t)> maxCount, bool fullSync) {
            IrTemplate t;
            t.name = name;
            t.op = op;
            t.gen = std::move(gen);
            t.maxCountPerLoop = std::move(maxCount);
            t.fullSyncEachCall = fullSync;
            R.Register(t);
        };
        // scratch multiples (in units of the chunk payload): see the generators above
        reg("InsAllReduceMesh1DOneShot", HCCL_CMD_ALLREDUCE, GenAllReduceOneShot,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("InsAllReduceMesh1DTwoShot", HCCL_CMD_ALLREDUCE, GenAllReduceTwoShot,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 1.0 + 1.0 / n); }, true);
        reg("InsAllReduceRing", HCCL_CMD_ALLREDUCE, GenAllReduceRing,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 2.0 * (n - 1) / n + 1e-9); }, true);
        reg("InsAllReduceNHR", HCCL_CMD_ALLREDUCE, GenAllReduceNhr,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 2.0 * NhrStageSlices(n) / n + 1e-9); }, true);
        reg("InsAllGatherMesh1D", HCCL_CMD_ALLGATHER, GenAllGatherMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 1.0); }, true);
        reg("InsAllGatherRing", HCCL_CMD_ALLGATHER, GenAllGatherRing,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)std::max(1u, n - 1)); }, true);
        reg("InsAllGatherNHR", HCCL_CMD_ALLGATHER, GenAllGatherNhr,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)std::max<uint64_t>(1, NhrStageSlices(n))); }, true);
        reg("InsReduceScatterMesh1D", HCCL_CMD_REDUCE_SCATTER, GenReduceScatterMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("InsReduceScatterRing", HCCL_CMD_REDUCE_SCATTER, GenReduceScatterRing,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)std::max(1u, n - 1)); }, true);
        reg("InsReduceScatterNHR", HCCL_CMD_REDUCE_SCATTER, GenReduceScatterNhr,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)(n + NhrStageSlices(n))); }, true);
        reg("InsBroadcastMesh1DOneShot", HCCL_CMD_BROADCAST, GenBroadcastOneShot,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 1.0); }, true);
        reg("InsBroadcastMesh1DTwoShot", HCCL_CMD_BROADCAST, GenBroadcastTwoShot,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 1.0); }, true);
        reg("ReduceMesh1D", HCCL_CMD_REDUCE, GenReduceMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("ReduceMesh1DTwoShot", HCCL_CMD_REDUCE, GenReduceTwoShot,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 2.0 + 2.0 / n); }, true);
        reg("InsScatterMesh1D", HCCL_CMD_SCATTER, GenScatterMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("InsGatherMesh1D", HCCL_CMD_GATHER, GenGatherMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 1.0); }, true);
        reg("InsScatterNHR", HCCL_CMD_SCATTER, GenScatterNhr,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("InsBroadcastNHR", HCCL_CMD_BROADCAST, GenBroadcastNhr,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (1.0 + NhrStageSlices(n)) / n + 1e-9); }, true);
        reg("ReduceNHR", HCCL_CMD_REDUCE, GenReduceNhr,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (2.0 * n + NhrStageSlices(n)) / n + 1e-9); }, true);
        reg("InsAlltoAllMesh1D", HCCL_CMD_ALLTOALL, GenAlltoAllMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("InsAlltoAllVMesh1D", HCCL_CMD_ALLTOALLV, GenAlltoAllVMesh, Unlimited, true);
        reg("InsAlltoAllVCMesh1D", HCCL_CMD_ALLTOALLVC, GenAlltoAllVMesh, Unlimited, true);
        reg("InsAllGatherVMesh1D", HCCL_CMD_ALLGATHER_V, GenAllGatherVMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, 1.0); }, true);
        reg("InsReduceScatterVMesh1D", HCCL_CMD_REDUCE_SCATTER_V, GenReduceScatterVMesh,
            [](uint32_t n, uint32_t es, uint64_t ccl) { return PerN(n, es, ccl, (double)n); }, true);
        reg("InsBarrierMesh1D", HCCL_CMD_BARRIER, GenBarrierMesh, Unlimited, true);
        reg("InsBarrierNHR", HCCL_CMD_BARRIER, GenBarrierNhr, Unlimited, true);
    });
}

}  // namespace hccl
