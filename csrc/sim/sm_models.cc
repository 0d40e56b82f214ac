// Schedule models of the SM / NVLS collective kernels, in the IR the offline checker consumes.
//
// The kernels in csrc/kernels/collectives.cu are not issued task by task, so they have no schedule of their own to check.
// Each model here restates one kernel body as IR, with the same arithmetic (128-byte aligned slots and slices, PartOf
// splitting over channels, rank rotation) and the same synchronisation points: a channel is a queue, a channel barrier
// is a POST to and a WAIT for every peer on that channel's slot, a plain peer store / load is a WRITE / READ, a rank-ordered
// slot reduction is a copy of slot 0 followed by LOCAL_REDUCE of the others, multimem.ld_reduce is a copy of the own scratch
// followed by READ_REDUCE of every peer's, multimem.st a copy plus a WRITE to every peer. The launch lists come from the real
// planner (SmPlanOp), so chunk loops and per-chunk offsets are the ones that run. With the models HcclCheckAlgorithm
// proves deadlock freedom, bounds, freedom from races and the operator's semantics for the default GPU engines too
// (the reference checks its generated task graphs the same way: test/st/algorithm/utils/src/hccl_verifier/checker.cc:50-100).
// The warp-specialised pipelined / push variants (pipelined.cuh) are modelled with three queues per channel (one per role
// group) and notifies between the queues of a rank; see the section on them below. Point-to-point kernels are not modelled
// here (their mailbox schedules are checked as host-issued plans).
#include <algorithm>
#include "../common/log.h"
#include "../kernels/coll_args.h"
#include "checker.h"

namespace hccl {

namespace {
uint64_t Up128(uint64_t v) { return (v + 127) & ~127ull; }
uint64_t SliceLen(uint64_t total, uint64_t slice, uint32_t j)
{
    uint64_t off = slice * (uint64_t)j;
    return off >= total ? 0 : std::min(slice, total - off);
}
struct Part { uint64_t off, len; };
Part PartOf(uint64_t total, uint32_t parts, uint32_t b)
{
    uint64_t per = ((total + parts - 1) / parts + 127) & ~127ull;
    uint64_t off = per * b;
    Part p;
    p.off = off < total ? off : total;
    p.len = off < total ? std::min(per, total - off) : 0;
    return p;
}

struct Model {
    const std::vector<SmLaunch> &all;    // this chunk's launch of every rank
    uint32_t me, n, C;
    uintptr_t inBase, outBase;
    bool inIsOutput;                     // Broadcast works in the output buffer
    Plan *plan;
    const CollArgs &A() const { return all[me].args; }
    BufRef In(uint64_t off) const
    {
        uintptr_t a = (uintptr_t)A().in + off;
        return a >= outBase ? BufRef{BufKind::OUTPUT, a - outBase} : BufRef{BufKind::INPUT, a - inBase};
    }
    BufRef Out(uint64_t off) const { return BufRef{BufKind::OUTPUT, (uintptr_t)A().out + off - outBase}; }
    static BufRef Ccl(uint64_t off) { return BufRef{BufKind::CCL, off}; }
    std::vector<Task> &Q(uint32_t ch) { return plan->queues[ch]; }
    void Copy(uint32_t ch, BufRef d, BufRef s, uint64_t len) { if (len) Q(ch).push_back(Task{TaskType::LOCAL_COPY, 0, 0, d, s, len}); }
    void Reduce(uint32_t ch, BufRef d, BufRef s, uint64_t len) { if (len) Q(ch).push_back(Task{TaskType::LOCAL_REDUCE, 0, 0, d, s, len}); }
    void Write(uint32_t ch, uint32_t peer, uint64_t cclOff, BufRef s, uint64_t len)
    {
        if (!len) return;
        if (peer == me) Copy(ch, Ccl(cclOff), s, len);
        else Q(ch).push_back(Task{TaskType::WRITE, peer, 0, Ccl(cclOff), s, len});
    }
    void WriteReduce(uint32_t ch, uint32_t peer, uint64_t cclOff, BufRef s, uint64_t len)
    {
        if (!len) return;
        if (peer == me) Reduce(ch, Ccl(cclOff), s, len);
        else Q(ch).push_back(Task{TaskType::WRITE_REDUCE, peer, 0, Ccl(cclOff), s, len});
    }
    void Read(uint32_t ch, BufRef d, uint32_t peer, uint64_t cclOff, uint64_t len)
    {
        if (!len) return;
        if (peer == me) Copy(ch, d, Ccl(cclOff), len);
        else Q(ch).push_back(Task{TaskType::READ, peer, 0, d, Ccl(cclOff), len});
    }
    void ReadReduce(uint32_t ch, BufRef d, uint32_t peer, uint64_t cclOff, uint64_t len)
    {
        if (!len) return;
        if (peer == me) Reduce(ch, d, Ccl(cclOff), len);
        else Q(ch).push_back(Task{TaskType::READ_REDUCE, peer, 0, d, Ccl(cclOff), len});
    }
    void Post(uint32_t ch, uint32_t peer) { Q(ch).push_back(Task{TaskType::POST, peer, ch, {}, {}, 0}); }
    void Wait(uint32_t ch, uint32_t peer) { Q(ch).push_back(Task{TaskType::WAIT, peer, ch, {}, {}, 0}); }
    void Barrier(uint32_t ch)
    {
        for (uint32_t d = 1; d < n; ++d) Post(ch, (me + d) % n);
        for (uint32_t d = 1; d < n; ++d) Wait(ch, (me + d) % n);
    }
    // dst <- slot[0] (op) slot[1] ... in rank order; slots are in this rank's scratch
    void ReduceSlots(uint32_t ch, BufRef dst, uint64_t slot0, uint64_t stride, uint64_t len)
    {
        Copy(ch, dst, Ccl(slot0), len);
        for (uint32_t r = 1; r < n; ++r) Reduce(ch, dst, Ccl(slot0 + r * stride), len);
    }
    // dst <- switch reduction of every rank's scratch at cclOff
    void MultimemLdReduce(uint32_t ch, BufRef dst, uint64_t cclOff, uint64_t len)
    {
        Copy(ch, dst, Ccl(cclOff), len);
        for (uint32_t d = 1; d < n; ++d) ReadReduce(ch, dst, (me + d) % n, cclOff, len);
    }
    // every rank's scratch at cclOff <- src
    void MultimemSt(uint32_t ch, uint64_t cclOff, BufRef src, uint64_t len)
    {
        for (uint32_t d = 0; d < n; ++d) Write(ch, (me + d) % n, cclOff, src, len);
    }
};

void AllReduceOneShot(Model &m, bool nvls)
{
    const uint64_t bytes = m.A().bytes, slot = Up128(bytes);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Part p = PartOf(bytes, m.C, ch);
        if (nvls) {
            m.Copy(ch, Model::Ccl(p.off), m.In(p.off), p.len);
            m.Barrier(ch);
            m.MultimemLdReduce(ch, m.Out(p.off), p.off, p.len);
        } else {
            for (uint32_t d = 0; d < m.n; ++d) m.Write(ch, (m.me + d) % m.n, (uint64_t)m.me * slot + p.off, m.In(p.off), p.len);
            m.Barrier(ch);
            m.ReduceSlots(ch, m.Out(p.off), p.off, slot, p.len);
        }
    }
}

void AllReduceTwoShot(Model &m, bool nvls)
{
    const uint32_t n = m.n;
    const uint64_t bytes = m.A().bytes, slice = Up128((bytes + n - 1) / n), outRegion = (uint64_t)n * slice;
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        if (nvls) {
            for (uint32_t j = 0; j < n; ++j) { Part p = PartOf(SliceLen(bytes, slice, j), m.C, ch); m.Copy(ch, Model::Ccl(j * slice + p.off), m.In(j * slice + p.off), p.len); }
            m.Barrier(ch);
            Part p = PartOf(SliceLen(bytes, slice, m.me), m.C, ch);
            // reduced slice -> every rank's result region (multimem.ld_reduce then multimem.st)
            m.MultimemLdReduce(ch, Model::Ccl(outRegion + m.me * slice + p.off), m.me * slice + p.off, p.len);
            for (uint32_t d = 1; d < n; ++d) m.Write(ch, (m.me + d) % n, outRegion + m.me * slice + p.off, Model::Ccl(outRegion + m.me * slice + p.off), p.len);
            m.Barrier(ch);
            for (uint32_t j = 0; j < n; ++j) { Part q = PartOf(SliceLen(bytes, slice, j), m.C, ch); m.Copy(ch, m.Out(j * slice + q.off), Model::Ccl(outRegion + j * slice + q.off), q.len); }
        } else {
            for (uint32_t d = 0; d < n; ++d) {
                uint32_t r = (m.me + d) % n;
                Part p = PartOf(SliceLen(bytes, slice, r), m.C, ch);
                m.Write(ch, r, (uint64_t)m.me * slice + p.off, m.In((uint64_t)r * slice + p.off), p.len);
            }
            m.Barrier(ch);
            Part p = PartOf(SliceLen(bytes, slice, m.me), m.C, ch);
            m.ReduceSlots(ch, Model::Ccl(outRegion + p.off), p.off, slice, p.len);
            m.Copy(ch, m.Out((uint64_t)m.me * slice + p.off), Model::Ccl(outRegion + p.off), p.len);
            m.Barrier(ch);
            for (uint32_t d = 1; d < n; ++d) {
                uint32_t r = (m.me + d) % n;
                Part q = PartOf(SliceLen(bytes, slice, r), m.C, ch);
                m.Read(ch, m.Out((uint64_t)r * slice + q.off), r, outRegion + q.off, q.len);
            }
        }
    }
}

// Two sub-grids: channels [0, splitCtas) run the first algorithm on the first splitBytes, the rest the peer-store two-shot on
// the remainder, in a scratch region shifted past part A's.
void AllReduceConcurrent(Model &m, bool nvls)
{
    const uint32_t n = m.n;
    const CollArgs &A = m.A();
    const uint64_t bytesA = A.splitBytes, bytesB = A.bytes - bytesA;
    // the model keeps the launch's proportion of CTAs, with at least one channel per part
    const uint32_t ca = std::max(1u, std::min(m.C - 1, (uint32_t)((uint64_t)m.C * A.splitCtas / std::max(1u, m.all[m.me].ctas))));
    const uint64_t shift = 2ull * n * Up128((bytesA + n - 1) / n);
    auto twoShot = [&](uint32_t ch, uint32_t vb, uint32_t vg, uint64_t base, uint64_t io, uint64_t bytes, bool viaSwitch) {
        const uint64_t slice = Up128((bytes + n - 1) / n), outRegion = (uint64_t)n * slice;
        if (viaSwitch) {
            for (uint32_t j = 0; j < n; ++j) { Part p = PartOf(SliceLen(bytes, slice, j), vg, vb); m.Copy(ch, Model::Ccl(base + j * slice + p.off), m.In(io + j * slice + p.off), p.len); }
            m.Barrier(ch);
            Part p = PartOf(SliceLen(bytes, slice, m.me), vg, vb);
            m.MultimemLdReduce(ch, Model::Ccl(base + outRegion + m.me * slice + p.off), base + m.me * slice + p.off, p.len);
            for (uint32_t d = 1; d < n; ++d) m.Write(ch, (m.me + d) % n, base + outRegion + m.me * slice + p.off, Model::Ccl(base + outRegion + m.me * slice + p.off), p.len);
            m.Barrier(ch);
            for (uint32_t j = 0; j < n; ++j) { Part q = PartOf(SliceLen(bytes, slice, j), vg, vb); m.Copy(ch, m.Out(io + j * slice + q.off), Model::Ccl(base + outRegion + j * slice + q.off), q.len); }
        } else {
            for (uint32_t d = 0; d < n; ++d) {
                uint32_t r = (m.me + d) % n;
                Part p = PartOf(SliceLen(bytes, slice, r), vg, vb);
                m.Write(ch, r, base + (uint64_t)m.me * slice + p.off, m.In(io + (uint64_t)r * slice + p.off), p.len);
            }
            m.Barrier(ch);
            Part p = PartOf(SliceLen(bytes, slice, m.me), vg, vb);
            m.ReduceSlots(ch, Model::Ccl(base + outRegion + p.off), base + p.off, slice, p.len);
            m.Copy(ch, m.Out(io + (uint64_t)m.me * slice + p.off), Model::Ccl(base + outRegion + p.off), p.len);
            m.Barrier(ch);
            for (uint32_t d = 1; d < n; ++d) {
                uint32_t r = (m.me + d) % n;
                Part q = PartOf(SliceLen(bytes, slice, r), vg, vb);
                m.Read(ch, m.Out(io + (uint64_t)r * slice + q.off), r, base + outRegion + q.off, q.len);
            }
        }
    };
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        if (ch < ca) twoShot(ch, ch, ca, 0, 0, bytesA, nvls);
        else twoShot(ch, ch - ca, m.C - ca, shift, bytesA, bytesB, false);
    }
}

void AllReduceRing(Model &m)
{
    const uint32_t n = m.n, next = (m.me + 1) % n, prev = (m.me + n - 1) % n;
    const uint64_t bytes = m.A().bytes, slice = Up128((bytes + n - 1) / n);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        auto part = [&](uint32_t j) { return PartOf(SliceLen(bytes, slice, j), m.C, ch); };
        for (uint32_t s = 0; s + 1 < n; ++s) {
            const uint32_t j = (m.me + n - s) % n;
            Part p = part(j);
            if (s == 0) m.Write(ch, next, p.off, m.In(j * slice + p.off), p.len);
            else {
                m.Wait(ch, prev);
                m.Write(ch, next, s * slice + p.off, Model::Ccl((s - 1) * slice + p.off), p.len);
                m.WriteReduce(ch, next, s * slice + p.off, m.In(j * slice + p.off), p.len);
            }
            m.Post(ch, next);
        }
        {
            m.Wait(ch, prev);
            const uint32_t j = (m.me + 1) % n;
            Part p = part(j);
            m.Copy(ch, m.Out(j * slice + p.off), Model::Ccl((uint64_t)(n - 2) * slice + p.off), p.len);
            m.Reduce(ch, m.Out(j * slice + p.off), m.In(j * slice + p.off), p.len);
            m.Write(ch, next, (uint64_t)(n - 1) * slice + p.off, m.Out(j * slice + p.off), p.len);
            m.Post(ch, next);
        }
        for (uint32_t a = 1; a < n; ++a) {
            m.Wait(ch, prev);
            const uint32_t j = (m.me + 1 + n - a) % n;
            Part p = part(j);
            const uint64_t got = (uint64_t)(n - 2 + a) * slice + p.off;
            m.Copy(ch, m.Out(j * slice + p.off), Model::Ccl(got), p.len);
            if (a + 1 < n) { m.Write(ch, next, (uint64_t)(n - 1 + a) * slice + p.off, Model::Ccl(got), p.len); m.Post(ch, next); }
        }
    }
}

void AllGatherV(Model &m)
{
    const CollArgs &A = m.A();
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Part p = PartOf(A.recvBytes[m.me], m.C, ch);
        m.Copy(ch, Model::Ccl(p.off), m.In(p.off), p.len);
        m.Barrier(ch);
        for (uint32_t d = 1; d < m.n; ++d) {
            uint32_t r = (m.me + d) % m.n;
            Part q = PartOf(A.recvBytes[r], m.C, ch);
            m.Read(ch, m.Out(A.recvOff[r] + q.off), r, q.off, q.len);
        }
        m.Copy(ch, m.Out(A.recvOff[m.me] + p.off), m.In(p.off), p.len);
    }
}

void ReduceScatterV(Model &m, bool nvls)
{
    const CollArgs &A = m.A();
    uint64_t slot = 0;
    if (nvls) slot = Up128(A.sendBytes[0]);
    else { for (uint32_t r = 0; r < m.n; ++r) slot = std::max(slot, A.sendBytes[r]); slot = Up128(slot); }
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        if (nvls) {
            for (uint32_t j = 0; j < m.n; ++j) { Part p = PartOf(A.sendBytes[j], m.C, ch); m.Copy(ch, Model::Ccl(j * slot + p.off), m.In(A.sendOff[j] + p.off), p.len); }
            m.Barrier(ch);
            Part p = PartOf(A.sendBytes[m.me], m.C, ch);
            m.MultimemLdReduce(ch, m.Out(p.off), (uint64_t)m.me * slot + p.off, p.len);
        } else {
            for (uint32_t d = 0; d < m.n; ++d) {
                uint32_t r = (m.me + d) % m.n;
                Part p = PartOf(A.sendBytes[r], m.C, ch);
                m.Write(ch, r, (uint64_t)m.me * slot + p.off, m.In(A.sendOff[r] + p.off), p.len);
            }
            m.Barrier(ch);
            Part p = PartOf(A.sendBytes[m.me], m.C, ch);
            m.ReduceSlots(ch, m.Out(p.off), p.off, slot, p.len);
        }
    }
}

void Broadcast(Model &m, bool nvls)
{
    const CollArgs &A = m.A();
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Part p = PartOf(A.bytes, m.C, ch);
        if (m.me == A.root) { if (nvls) m.MultimemSt(ch, p.off, m.In(p.off), p.len); else m.Copy(ch, Model::Ccl(p.off), m.In(p.off), p.len); }
        m.Barrier(ch);
        if (m.me != A.root) { if (nvls) m.Copy(ch, m.Out(p.off), Model::Ccl(p.off), p.len); else m.Read(ch, m.Out(p.off), A.root, p.off, p.len); }
    }
}

void ReduceToRoot(Model &m)
{
    const CollArgs &A = m.A();
    const uint64_t slot = Up128(A.bytes);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Part p = PartOf(A.bytes, m.C, ch);
        m.Write(ch, A.root, (uint64_t)m.me * slot + p.off, m.In(p.off), p.len);
        m.Barrier(ch);
        if (m.me == A.root) m.ReduceSlots(ch, m.Out(p.off), p.off, slot, p.len);
    }
}

void Scatter(Model &m)
{
    const CollArgs &A = m.A();
    const uint64_t slot = Up128(A.bytes);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Part p = PartOf(A.bytes, m.C, ch);
        if (m.me == A.root)
            for (uint32_t r = 0; r < m.n; ++r) if (r != A.root) m.Copy(ch, Model::Ccl((uint64_t)r * slot + p.off), m.In(A.sendOff[r] + p.off), p.len);
        m.Barrier(ch);
        if (m.me == A.root) m.Copy(ch, m.Out(p.off), m.In(A.sendOff[A.root] + p.off), p.len);
        else m.Read(ch, m.Out(p.off), A.root, (uint64_t)m.me * slot + p.off, p.len);
    }
}

// ---- zero-copy forms: peers address the registered user windows directly (remote INPUT / OUTPUT references)
void ZcPeerRead(Model &m, uint32_t ch, BufRef dst, uint32_t peer, BufRef src, uint64_t len, bool reduce)
{
    if (!len) return;
    if (peer == m.me) { if (reduce) m.Reduce(ch, dst, src, len); else m.Copy(ch, dst, src, len); }
    else m.Q(ch).push_back(Task{reduce ? TaskType::READ_REDUCE : TaskType::READ, peer, 0, dst, src, len});
}
void ZcPeerWrite(Model &m, uint32_t ch, uint32_t peer, BufRef dst, BufRef src, uint64_t len)
{
    if (!len) return;
    if (peer == m.me) { if (!(dst.kind == src.kind && dst.off == src.off)) m.Copy(ch, dst, src, len); }
    else m.Q(ch).push_back(Task{TaskType::WRITE, peer, 0, dst, src, len});
}
void AllReduceZc(Model &m)
{
    const uint32_t n = m.n;
    const uint64_t bytes = m.A().bytes, slice = Up128((bytes + n - 1) / n);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        m.Barrier(ch);
        Part p = PartOf(SliceLen(bytes, slice, m.me), m.C, ch);
        const uint64_t so = (uint64_t)m.me * slice + p.off;
        // the owner's reduction of its slice lands in its own output first, then goes to every peer's output
        for (uint32_t r = 0; r < n; ++r) ZcPeerRead(m, ch, m.Out(so), r, m.In(so), p.len, r != 0);
        for (uint32_t d = 1; d < n; ++d) ZcPeerWrite(m, ch, (m.me + d) % n, m.Out(so), m.Out(so), p.len);
        m.Barrier(ch);
    }
}
void ReduceScatterZc(Model &m)
{
    const uint64_t bytes = m.A().bytes;
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        m.Barrier(ch);
        Part p = PartOf(bytes, m.C, ch);
        for (uint32_t r = 0; r < m.n; ++r) ZcPeerRead(m, ch, m.Out(p.off), r, m.In((uint64_t)m.me * bytes + p.off), p.len, r != 0);
        m.Barrier(ch);
    }
}
void AllGatherZc(Model &m)
{
    const uint64_t bytes = m.A().bytes;
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        m.Barrier(ch);
        Part p = PartOf(bytes, m.C, ch);
        for (uint32_t d = 0; d < m.n; ++d) ZcPeerWrite(m, ch, (m.me + d) % m.n, m.Out((uint64_t)m.me * bytes + p.off), m.In(p.off), p.len);
        m.Barrier(ch);
    }
}
void BroadcastZc(Model &m, bool nvls)
{
    const CollArgs &A = m.A();
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        m.Barrier(ch);
        Part p = PartOf(A.bytes, m.C, ch);
        if (nvls) { if (m.me == A.root) for (uint32_t d = 1; d < m.n; ++d) ZcPeerWrite(m, ch, (m.me + d) % m.n, m.Out(p.off), m.Out(p.off), p.len); }
        else if (m.me != A.root) ZcPeerRead(m, ch, m.Out(p.off), A.root, m.Out(p.off), p.len, false);
        m.Barrier(ch);
    }
}

// Fixed slot per (source, destination) pair, rounds of slotBytes, the same number of rounds on every rank (the kernel
// takes the maximum over all ranks' rows and columns).
void AlltoAllV(Model &m)
{
    const CollArgs &A = m.A();
    const uint64_t Q = A.slotBytes;
    uint64_t R = 0;
    for (uint32_t a = 0; a < m.n; ++a)
        for (uint32_t r = 0; r < m.n; ++r)
            if (r != a) R = std::max(R, (std::max(m.all[a].args.sendBytes[r], m.all[a].args.recvBytes[r]) + Q - 1) / Q);
    auto slotOf = [&](uint32_t owner, uint32_t dst) { return (uint64_t)(dst < owner ? dst : dst - 1) * Q; };
    // the kernel's PartOfRound: the first round of a pair fixes which bytes of the slot a channel owns
    auto partAt = [&](uint64_t total, uint64_t t, uint32_t ch) {
        const uint64_t first = std::min(total, Q), per = ((first + m.C - 1) / m.C + 127) & ~127ull;
        const uint64_t len = total <= t * Q ? 0 : std::min(Q, total - t * Q), off = per * ch;
        Part p;
        p.off = off < len ? off : len;
        p.len = off < len ? std::min(len - off, per) : 0;
        return p;
    };
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Part self = PartOf(A.sendBytes[m.me], m.C, ch);
        m.Copy(ch, m.Out(A.recvOff[m.me] + self.off), m.In(A.sendOff[m.me] + self.off), self.len);
        auto stage = [&](uint64_t t) {
            for (uint32_t r = 0; r < m.n; ++r) {
                if (r == m.me) continue;
                Part p = partAt(A.sendBytes[r], t, ch);
                m.Copy(ch, Model::Ccl(slotOf(m.me, r) + p.off), m.In(A.sendOff[r] + t * Q + p.off), p.len);
            }
        };
        stage(0);
        m.Barrier(ch);
        for (uint64_t t = 0; t < R; ++t) {
            if (t > 0) { stage(t); m.Barrier(ch); }
            for (uint32_t d = 1; d < m.n; ++d) {
                uint32_t r = (m.me + d) % m.n;
                Part p = partAt(A.recvBytes[r], t, ch);
                m.Read(ch, m.Out(A.recvOff[r] + t * Q + p.off), r, slotOf(r, m.me) + p.off, p.len);
            }
            if (t + 1 < R) m.Barrier(ch);
        }
    }
}
// ---------------------------------------------------------------------------------------------- warp-specialised pipelines
// pipelined.cuh: every CTA is a channel with role groups (stagers / movers / drainers) that walk the channel's sub-chunks
// through rings of kPipeDepth slots and meet through three monotonic per-channel counters (STAGED, MOVED, DRAINED) that
// every rank raises on every rank. Here a role group is a queue (3 per channel), "all ranks have raised X to c + 1" is a
// WAIT for the next notify of every peer plus a local wait for the own producer group, and a signal is posted once per
// consumer group and only for the chunks that group will wait for (the counters are level-triggered, notifies are counted).
// The geometry (slices, PartOf, sub-chunk count = the channel's LONGEST part over all slices, slot addresses) restates the
// kernel's, with the launch's own grid and sub-chunk size.
constexpr uint32_t kPipeDepth = 2;
enum PipeRole : uint32_t { ROLE_A = 0, ROLE_B = 1, ROLE_C = 2 };
enum PipeSlot : uint32_t { S_STAGED_MOVER = 0, S_MOVED_STAGER = 1, S_MOVED_DRAINER = 2, S_DRAINED_MOVER = 3 };

struct Pipe {
    Model &m;
    uint32_t ch, G;
    uint64_t sub;
    uint32_t chunks;
    uint32_t Q(PipeRole r) const { return ch * 3 + r; }
    uint64_t Slot(uint32_t d, uint32_t j) const { return (((uint64_t)d * m.n + j) * G + ch) * sub; }
    uint64_t RingBytes() const { return (uint64_t)kPipeDepth * m.n * G * sub; }
    static uint64_t SubLen(uint64_t len, uint64_t sub, uint32_t c) { uint64_t lo = (uint64_t)c * sub; return lo >= len ? 0 : std::min(sub, len - lo); }
    std::vector<Task> &Tasks(PipeRole r) { return m.plan->queues[Q(r)]; }
    void Signal(PipeRole from, PipeSlot slot, PipeRole consumer)
    {
        for (uint32_t d = 1; d < m.n; ++d) Tasks(from).push_back(Task{TaskType::POST, (m.me + d) % m.n, ch * 8 + slot, {}, {}, 0});
        Tasks(from).push_back(Task{TaskType::LOCAL_POST, Q(consumer), 0, {}, {}, 0});
    }
    void Wait(PipeRole at, PipeSlot slot, PipeRole producer)
    {
        for (uint32_t d = 1; d < m.n; ++d) Tasks(at).push_back(Task{TaskType::WAIT, (m.me + d) % m.n, ch * 8 + slot, {}, {}, 0});
        Tasks(at).push_back(Task{TaskType::LOCAL_WAIT, Q(producer), 0, {}, {}, 0});
    }
    void Copy(PipeRole r, BufRef d, BufRef s, uint64_t len) { if (len) Tasks(r).push_back(Task{TaskType::LOCAL_COPY, 0, 0, d, s, len}); }
    // dst (local) <- every rank's scratch at cclOff, combined in rank order
    void GatherReduce(PipeRole r, BufRef dst, uint64_t cclOff, uint64_t len)
    {
        if (!len) return;
        for (uint32_t q = 0; q < m.n; ++q) {
            const bool first = q == 0;
            if (q == m.me) Tasks(r).push_back(Task{first ? TaskType::LOCAL_COPY : TaskType::LOCAL_REDUCE, 0, 0, dst, Model::Ccl(cclOff), len});
            else Tasks(r).push_back(Task{first ? TaskType::READ : TaskType::READ_REDUCE, q, 0, dst, Model::Ccl(cclOff), len});
        }
    }
    void WriteTo(PipeRole r, uint32_t peer, uint64_t cclOff, BufRef src, uint64_t len)
    {
        if (!len) return;
        if (peer == m.me) Copy(r, Model::Ccl(cclOff), src, len);
        else Tasks(r).push_back(Task{TaskType::WRITE, peer, 0, Model::Ccl(cclOff), src, len});
    }
};

Pipe MakePipe(Model &m, uint32_t ch, const std::vector<uint64_t> &blockBytes)
{
    const CollArgs &A = m.A();
    Pipe p{m, ch, m.C, A.pipeSub, 0};
    uint64_t longest = 0;
    for (uint64_t b : blockBytes) longest = std::max(longest, PartOf(b, m.C, ch).len);
    p.chunks = (uint32_t)((longest + p.sub - 1) / p.sub);
    return p;
}

void AllReducePipe(Model &m)
{
    const CollArgs &A = m.A();
    const uint64_t bytes = A.bytes, slice = Up128((bytes + m.n - 1) / m.n);
    std::vector<uint64_t> lens(m.n);
    for (uint32_t j = 0; j < m.n; ++j) lens[j] = SliceLen(bytes, slice, j);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Pipe p = MakePipe(m, ch, lens);
        const uint64_t resBase = p.RingBytes();
        const Part mine = PartOf(lens[m.me], m.C, ch);
        for (uint32_t c = 0; c < p.chunks; ++c) {
            const uint32_t d = c % kPipeDepth;
            const bool reused = c + kPipeDepth < p.chunks;                 // somebody will wait for this chunk's slot to be free again
            // stagers: input -> staging ring, one slot per destination slice
            if (c >= kPipeDepth) p.Wait(ROLE_A, S_MOVED_STAGER, ROLE_B);
            for (uint32_t j = 0; j < m.n; ++j) {
                Part pj = PartOf(lens[j], m.C, ch);
                p.Copy(ROLE_A, Model::Ccl(p.Slot(d, j)), m.In((uint64_t)j * slice + pj.off + (uint64_t)c * p.sub), Pipe::SubLen(pj.len, p.sub, c));
            }
            p.Signal(ROLE_A, S_STAGED_MOVER, ROLE_B);
            // movers: reduce the own slice over all ranks' staging slots, store the result into every rank's result ring
            p.Wait(ROLE_B, S_STAGED_MOVER, ROLE_A);
            if (c >= kPipeDepth) p.Wait(ROLE_B, S_DRAINED_MOVER, ROLE_C);
            const uint64_t len = Pipe::SubLen(mine.len, p.sub, c), res = resBase + p.Slot(d, m.me);
            p.GatherReduce(ROLE_B, Model::Ccl(res), p.Slot(d, m.me), len);
            for (uint32_t q = 1; q < m.n; ++q) p.WriteTo(ROLE_B, (m.me + q) % m.n, res, Model::Ccl(res), len);
            if (reused) p.Signal(ROLE_B, S_MOVED_STAGER, ROLE_A);
            p.Signal(ROLE_B, S_MOVED_DRAINER, ROLE_C);
            // drainers: result ring -> output
            p.Wait(ROLE_C, S_MOVED_DRAINER, ROLE_B);
            for (uint32_t j = 0; j < m.n; ++j) {
                Part pj = PartOf(lens[j], m.C, ch);
                p.Copy(ROLE_C, m.Out((uint64_t)j * slice + pj.off + (uint64_t)c * p.sub), Model::Ccl(resBase + p.Slot(d, j)), Pipe::SubLen(pj.len, p.sub, c));
            }
            if (reused) p.Signal(ROLE_C, S_DRAINED_MOVER, ROLE_B);
        }
    }
}

void ReduceScatterPipe(Model &m)
{
    const CollArgs &A = m.A();
    std::vector<uint64_t> lens(A.sendBytes, A.sendBytes + m.n);
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Pipe p = MakePipe(m, ch, lens);
        const Part mine = PartOf(lens[m.me], m.C, ch);
        for (uint32_t c = 0; c < p.chunks; ++c) {
            const uint32_t d = c % kPipeDepth;
            const bool reused = c + kPipeDepth < p.chunks;
            if (c >= kPipeDepth) p.Wait(ROLE_A, S_MOVED_STAGER, ROLE_B);
            for (uint32_t j = 0; j < m.n; ++j) {
                Part pj = PartOf(lens[j], m.C, ch);
                p.Copy(ROLE_A, Model::Ccl(p.Slot(d, j)), m.In(A.sendOff[j] + pj.off + (uint64_t)c * p.sub), Pipe::SubLen(pj.len, p.sub, c));
            }
            p.Signal(ROLE_A, S_STAGED_MOVER, ROLE_B);
            p.Wait(ROLE_B, S_STAGED_MOVER, ROLE_A);
            p.GatherReduce(ROLE_B, m.Out(mine.off + (uint64_t)c * p.sub), p.Slot(d, m.me), Pipe::SubLen(mine.len, p.sub, c));
            if (reused) p.Signal(ROLE_B, S_MOVED_STAGER, ROLE_A);
        }
    }
}

// AllGather(V), Broadcast as a one-contributor gather, and (a2a) AlltoAll with uniform counts: movers push, drainers copy out
void AllGatherPipe(Model &m, bool a2a)
{
    const CollArgs &A = m.A();
    std::vector<uint64_t> lens(A.recvBytes, A.recvBytes + m.n);
    const bool inPlace = !a2a && (uintptr_t)A.in == (uintptr_t)A.out + A.recvOff[m.me];
    for (uint32_t ch = 0; ch < m.C; ++ch) {
        Pipe p = MakePipe(m, ch, lens);
        const Part mine = PartOf(lens[m.me], m.C, ch);
        for (uint32_t c = 0; c < p.chunks; ++c) {
            const uint32_t d = c % kPipeDepth;
            const bool reused = c + kPipeDepth < p.chunks;
            if (c >= kPipeDepth) p.Wait(ROLE_A, S_DRAINED_MOVER, ROLE_B);
            for (uint32_t q = 0; q < m.n; ++q) {
                const uint32_t dst = (m.me + q) % m.n;
                if (a2a) {
                    Part ps = PartOf(A.sendBytes[dst], m.C, ch);
                    p.WriteTo(ROLE_A, dst, p.Slot(d, m.me), m.In(A.sendOff[dst] + ps.off + (uint64_t)c * p.sub), Pipe::SubLen(ps.len, p.sub, c));
                } else if (mine.len) {
                    p.WriteTo(ROLE_A, dst, p.Slot(d, m.me), m.In(mine.off + (uint64_t)c * p.sub), Pipe::SubLen(mine.len, p.sub, c));
                }
            }
            p.Signal(ROLE_A, S_MOVED_DRAINER, ROLE_B);
            p.Wait(ROLE_B, S_MOVED_DRAINER, ROLE_A);
            for (uint32_t q = 0; q < m.n; ++q) {
                const uint32_t j = (m.me + q) % m.n;
                if (j == m.me && inPlace) continue;
                Part pj = PartOf(lens[j], m.C, ch);
                p.Copy(ROLE_B, m.Out(A.recvOff[j] + pj.off + (uint64_t)c * p.sub), Model::Ccl(p.Slot(d, j)), Pipe::SubLen(pj.len, p.sub, c));
            }
            if (reused) p.Signal(ROLE_B, S_DRAINED_MOVER, ROLE_A);
        }
    }
}
}  // namespace

// Model of rank `me`'s kernel for one chunk. `all` = that chunk's launch on every rank (the V forms read peers' counts);
// inBase / outBase = the fake addresses the launches were planned with; channels = CTAs to model (the real grid only changes
// how finely the same byte ranges are split).
HcclResult GenSmModelPlan(const std::vector<SmLaunch> &all, uint32_t me, uintptr_t inBase, uintptr_t outBase, uint32_t channels, Plan *out)
{
    Model m{all, me, (uint32_t)all.size(), std::max(1u, channels), inBase, outBase, false, out};
    const SmKernelId kid = all[me].kernel;
    const bool pipelined = kid == K_ALLREDUCE_PIPE || kid == K_ALLREDUCE_PIPE_NVLS || kid == K_REDUCESCATTER_PIPE || kid == K_REDUCESCATTER_PIPE_NVLS ||
                           kid == K_ALLGATHER_PIPE || kid == K_ALLGATHER_PIPE_NVLS || kid == K_ALLTOALL_PIPE;
    if (pipelined) m.C = std::max(1u, all[me].ctas);      // slot addresses and the sub-chunk size depend on the grid: model the launch's own
    out->queues.clear();
    out->EnsureQueues(pipelined ? m.C * 3 : m.C);
    out->dtype = all[me].dtype;
    out->op = (HcclReduceOp)all[me].args.op;
    switch (all[me].kernel) {
        case K_ALLREDUCE_ONESHOT: AllReduceOneShot(m, false); break;
        case K_ALLREDUCE_NVLS_ONESHOT: AllReduceOneShot(m, true); break;
        case K_ALLREDUCE_TWOSHOT: AllReduceTwoShot(m, false); break;
        case K_ALLREDUCE_NVLS_TWOSHOT: AllReduceTwoShot(m, true); break;
        case K_ALLREDUCE_RING: AllReduceRing(m); break;
        case K_ALLREDUCE_CONCURRENT: AllReduceConcurrent(m, false); break;
        case K_ALLREDUCE_CONCURRENT_NVLS: AllReduceConcurrent(m, true); break;
        case K_ALLREDUCE_ZC: case K_ALLREDUCE_ZC_NVLS: AllReduceZc(m); break;      // the switch-reduced form moves the same data
        case K_REDUCESCATTER_ZC: case K_REDUCESCATTER_ZC_NVLS: ReduceScatterZc(m); break;
        case K_ALLGATHER_ZC: case K_ALLGATHER_ZC_NVLS: AllGatherZc(m); break;
        case K_BROADCAST_ZC: BroadcastZc(m, false); break;
        case K_BROADCAST_ZC_NVLS: BroadcastZc(m, true); break;
        case K_ALLGATHER_V: AllGatherV(m); break;
        case K_REDUCESCATTER_V: ReduceScatterV(m, false); break;
        case K_REDUCESCATTER_NVLS: ReduceScatterV(m, true); break;
        case K_BROADCAST: Broadcast(m, false); break;
        case K_BROADCAST_NVLS: Broadcast(m, true); break;
        case K_REDUCE: ReduceToRoot(m); break;
        case K_SCATTER: Scatter(m); break;
        case K_ALLTOALL_V: AlltoAllV(m); break;
        case K_BARRIER: for (uint32_t ch = 0; ch < m.C; ++ch) m.Barrier(ch); break;
        case K_ALLREDUCE_PIPE: case K_ALLREDUCE_PIPE_NVLS: AllReducePipe(m); break;        // the switch forms move the same data
        case K_REDUCESCATTER_PIPE: case K_REDUCESCATTER_PIPE_NVLS: ReduceScatterPipe(m); break;
        case K_ALLGATHER_PIPE: case K_ALLGATHER_PIPE_NVLS: AllGatherPipe(m, false); break;
        case K_ALLTOALL_PIPE: AllGatherPipe(m, true); break;
        default:
            HCCL_ERROR("no schedule model for kernel %u (the point-to-point kernels are checked as host-issued mailbox plans)", (unsigned)all[me].kernel);
            return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
