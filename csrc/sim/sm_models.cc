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
// Not modelled: the warp-specialised pipelined / push variants (pipelined.cuh), whose sub-chunk credit protocol has no
// counterpart in this IR; they are covered by the emulated-rank tests with real data.
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
}  // namespace

// Model of rank `me`'s kernel for one chunk. `all` = that chunk's launch on every rank (the V forms read peers' counts);
// inBase / outBase = the fake addresses the launches were planned with; channels = CTAs to model (the real grid only changes
// how finely the same byte ranges are split).
HcclResult GenSmModelPlan(const std::vector<SmLaunch> &all, uint32_t me, uintptr_t inBase, uintptr_t outBase, uint32_t channels, Plan *out)
{
    Model m{all, me, (uint32_t)all.size(), std::max(1u, channels), inBase, outBase, false, out};
    out->queues.clear();
    out->EnsureQueues(m.C);
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
        default:
            HCCL_ERROR("no schedule model for kernel %u (the pipelined and point-to-point kernels are checked with emulated ranks)", (unsigned)all[me].kernel);
            return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
