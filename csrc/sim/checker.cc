#include "checker.h"
#include <algorithm>
#include <deque>
#include <map>
#include <sstream>
#include "../common/dtype.h"

namespace hccl {
namespace {

using Contrib = std::pair<uint32_t, uint64_t>;          // (source rank, element index in that rank's input)
using Value = std::vector<Contrib>;                      // sorted multiset of contributions

struct Access {
    uint32_t rank;          // owner of the memory
    int kind;               // BufKind
    uint64_t lo, hi;        // byte range
    bool write;
    std::vector<uint32_t> clock;
    uint32_t byRank, byQueue, taskIdx;
};

struct World {
    const CheckSpec &spec;
    uint32_t n;
    // symbolic memory: (rank, kind) -> element index -> value
    std::map<std::pair<uint32_t, int>, std::map<uint64_t, Value>> mem;
    explicit World(const CheckSpec &s) : spec(s), n(s.nranks) {}
    Value &At(uint32_t rank, int kind, uint64_t elem) { return mem[{rank, kind}][elem]; }
};

}  // namespace

uint64_t CheckInputElems(const CheckSpec &s, uint32_t rank)
{
    switch (s.op) {
        case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_ALLTOALL: case HCCL_CMD_SCATTER: return s.count * s.nranks;
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: { uint64_t t = 0; for (uint32_t j = 0; j < s.nranks; ++j) t += s.countMatrix[rank * s.nranks + j]; return t; }
        case HCCL_CMD_ALLGATHER_V: return s.countMatrix[rank];
        case HCCL_CMD_REDUCE_SCATTER_V: { uint64_t t = 0; for (uint32_t j = 0; j < s.nranks; ++j) t += s.countMatrix[j]; return t; }
        default: return s.count;
    }
}

uint64_t CheckOutputElems(const CheckSpec &s, uint32_t rank)
{
    switch (s.op) {
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLTOALL: return s.count * s.nranks;
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: { uint64_t t = 0; for (uint32_t j = 0; j < s.nranks; ++j) t += s.countMatrix[j * s.nranks + rank]; return t; }
        case HCCL_CMD_ALLGATHER_V: { uint64_t t = 0; for (uint32_t j = 0; j < s.nranks; ++j) t += s.countMatrix[j]; return t; }
        case HCCL_CMD_REDUCE_SCATTER_V: return s.countMatrix[rank];
        default: return s.count;
    }
}

namespace {
uint64_t InputElems(const CheckSpec &s, uint32_t rank) { return CheckInputElems(s, rank); }

std::string Where(uint32_t rank, size_t q, size_t idx, const Task &t)
{
    std::ostringstream os;
    os << "rank " << rank << " queue " << q << " task " << idx << " (" << TaskTypeName(t.type) << " peer " << t.rank << " slot " << t.slot << " bytes " << t.bytes << ")";
    return os.str();
}

bool HappensBefore(const std::vector<uint32_t> &a, const std::vector<uint32_t> &b)
{
    bool strict = false;
    for (size_t i = 0; i < a.size(); ++i) {
        if (a[i] > b[i]) return false;
        if (a[i] < b[i]) strict = true;
    }
    return strict;
}

}  // namespace

HcclResult CheckPlans(const CheckSpec &spec, const std::vector<std::vector<Plan>> &chunks, std::string *why)
{
    const uint32_t n = spec.nranks, es = spec.elemSize;
    World w(spec);
    auto fail = [&](const std::string &m) { if (why) *why = m; return HCCL_E_INTERNAL; };
    // initial symbolic contents: input element i of rank r is {(r, i)}; broadcast works in the OUTPUT buffer
    for (uint32_t r = 0; r < n; ++r) {
        const int kind = spec.op == HCCL_CMD_BROADCAST ? (int)BufKind::OUTPUT : (int)BufKind::INPUT;
        for (uint64_t i = 0; i < InputElems(spec, r); ++i) w.At(r, kind, i) = {{r, i}};
    }
    for (size_t ci = 0; ci < chunks.size(); ++ci) {
        const std::vector<Plan> &plans = chunks[ci];
        if (plans.size() != n) return fail("chunk does not have one plan per rank");
        size_t maxQ = 0;
        for (auto &p : plans) maxQ = std::max(maxQ, p.queues.size());
        const size_t lanes = n * maxQ;                                         // one vector-clock lane per (rank, queue)
        std::vector<std::vector<size_t>> pc(n, std::vector<size_t>(maxQ, 0));
        std::vector<std::vector<std::vector<uint32_t>>> clock(n, std::vector<std::vector<uint32_t>>(maxQ, std::vector<uint32_t>(lanes, 0)));
        std::map<std::tuple<uint32_t, uint32_t, uint32_t>, std::deque<std::vector<uint32_t>>> inflight;   // (dst, src, slot) -> clocks of pending posts
        std::map<std::tuple<uint32_t, uint32_t, uint32_t>, std::deque<std::vector<uint32_t>>> localInflight;   // (rank, waiting queue, posting queue)
        std::vector<Access> accesses;
        size_t remaining = 0;
        for (auto &p : plans) remaining += p.TaskCount();
        // which rank's buffer a reference names decides its size: `owner` is the rank whose memory is touched
        auto bounds = [&](const BufRef &b, uint64_t bytes, uint32_t owner) {
            switch (b.kind) {
                case BufKind::CCL: return b.off + bytes <= spec.cclBytes;
                case BufKind::MAILBOX: return spec.mailboxBytes == 0 || b.off + bytes <= spec.mailboxBytes * 2 * (uint64_t)n;
                case BufKind::INPUT: return b.off + bytes <= std::max<uint64_t>(CheckInputElems(spec, owner), spec.op == HCCL_CMD_BROADCAST ? spec.count : 0) * es;
                case BufKind::OUTPUT: return b.off + bytes <= CheckOutputElems(spec, owner) * es;
                default: return true;
            }
        };
        // absolute addresses of BatchSendRecv items -> (INPUT | OUTPUT, offset)
        auto resolve = [&](BufRef b) {
            if (b.kind != BufKind::ABS) return b;
            if (spec.absOutputBase && b.off >= spec.absOutputBase) return BufRef{BufKind::OUTPUT, b.off - spec.absOutputBase};
            if (spec.absInputBase && b.off >= spec.absInputBase) return BufRef{BufKind::INPUT, b.off - spec.absInputBase};
            return b;
        };
        while (remaining > 0) {
            bool progressed = false;
            for (uint32_t r = 0; r < n; ++r) {
                for (size_t q = 0; q < plans[r].queues.size(); ++q) {
                    const auto &queue = plans[r].queues[q];
                    while (pc[r][q] < queue.size()) {
                        Task t = queue[pc[r][q]];
                        t.dst = resolve(t.dst);
                        t.src = resolve(t.src);
                        std::vector<uint32_t> &ck = clock[r][q];
                        if (t.type == TaskType::WAIT) {
                            auto it = inflight.find({r, t.rank, t.slot});
                            if (it == inflight.end() || it->second.empty()) break;          // blocked
                            for (size_t i = 0; i < lanes; ++i) ck[i] = std::max(ck[i], it->second.front()[i]);
                            it->second.pop_front();
                        } else if (t.type == TaskType::LOCAL_WAIT) {
                            // notifies between the queues of one rank: (rank, waiting queue, posting queue)
                            if (t.rank >= plans[r].queues.size() || t.rank == q) return fail("LOCAL_WAIT on an invalid queue at " + Where(r, q, pc[r][q], t));
                            auto it = localInflight.find({r, (uint32_t)q, t.rank});
                            if (it == localInflight.end() || it->second.empty()) break;     // blocked
                            for (size_t i = 0; i < lanes; ++i) ck[i] = std::max(ck[i], it->second.front()[i]);
                            it->second.pop_front();
                        }
                        ck[r * maxQ + q]++;
                        if (t.type == TaskType::POST) {
                            if (t.rank >= n || t.rank == r) return fail("POST to an invalid rank at " + Where(r, q, pc[r][q], t));
                            inflight[{t.rank, r, t.slot}].push_back(ck);
                        } else if (t.type == TaskType::LOCAL_POST) {
                            if (t.rank >= plans[r].queues.size() || t.rank == q) return fail("LOCAL_POST to an invalid queue at " + Where(r, q, pc[r][q], t));
                            localInflight[{r, t.rank, (uint32_t)q}].push_back(ck);
                        } else if (t.type != TaskType::WAIT && t.type != TaskType::LOCAL_WAIT) {
                            if (t.bytes % es) return fail("transfer is not a whole number of elements at " + Where(r, q, pc[r][q], t));
                            const bool remoteDst = t.type == TaskType::WRITE || t.type == TaskType::WRITE_REDUCE;
                            const bool remoteSrc = t.type == TaskType::READ || t.type == TaskType::READ_REDUCE;
                            const bool reduce = t.type == TaskType::LOCAL_REDUCE || t.type == TaskType::WRITE_REDUCE || t.type == TaskType::READ_REDUCE;
                            const uint32_t dstRank = remoteDst ? t.rank : r, srcRank = remoteSrc ? t.rank : r;
                            if (dstRank >= n || srcRank >= n) return fail("transfer names an invalid rank at " + Where(r, q, pc[r][q], t));
                            for (const BufRef *b : {&t.dst, &t.src})
                                if (!bounds(*b, t.bytes, b == &t.dst ? dstRank : srcRank))
                                    return fail(std::string(b->kind == BufKind::CCL ? "scratch window" : b->kind == BufKind::MAILBOX ? "mailbox" : "user buffer") +
                                                " overrun at " + Where(r, q, pc[r][q], t));
                            if (!spec.registeredUserBuffers &&
                                ((remoteDst && t.dst.kind != BufKind::CCL && t.dst.kind != BufKind::MAILBOX) || (remoteSrc && t.src.kind != BufKind::CCL && t.src.kind != BufKind::MAILBOX)))
                                return fail("remote access outside the symmetric heap at " + Where(r, q, pc[r][q], t));
                            accesses.push_back({srcRank, (int)t.src.kind, t.src.off, t.src.off + t.bytes, false, ck, r, (uint32_t)q, (uint32_t)pc[r][q]});
                            accesses.push_back({dstRank, (int)t.dst.kind, t.dst.off, t.dst.off + t.bytes, true, ck, r, (uint32_t)q, (uint32_t)pc[r][q]});
                            if (reduce) accesses.push_back({dstRank, (int)t.dst.kind, t.dst.off, t.dst.off + t.bytes, false, ck, r, (uint32_t)q, (uint32_t)pc[r][q]});
                            // symbolic execution
                            if (t.dst.off % es || t.src.off % es) return fail("unaligned element access at " + Where(r, q, pc[r][q], t));
                            for (uint64_t e = 0; e < t.bytes / es; ++e) {
                                Value v = w.At(srcRank, (int)t.src.kind, t.src.off / es + e);
                                Value &d = w.At(dstRank, (int)t.dst.kind, t.dst.off / es + e);
                                if (reduce) { d.insert(d.end(), v.begin(), v.end()); std::sort(d.begin(), d.end()); }
                                else d = v;
                            }
                        }
                        ++pc[r][q];
                        --remaining;
                        progressed = true;
                    }
                }
            }
            if (!progressed) {
                std::ostringstream os;
                os << "deadlock in chunk " << ci << ": blocked at";
                for (uint32_t r = 0; r < n; ++r)
                    for (size_t q = 0; q < plans[r].queues.size(); ++q)
                        if (pc[r][q] < plans[r].queues[q].size()) os << " [" << Where(r, q, pc[r][q], plans[r].queues[q][pc[r][q]]) << "]";
                return fail(os.str());
            }
        }
        for (auto &kv : inflight)
            if (!kv.second.empty()) {
                std::ostringstream os;
                os << "chunk " << ci << ": " << kv.second.size() << " notify(s) from rank " << std::get<1>(kv.first) << " to rank " << std::get<0>(kv.first) << " slot "
                   << std::get<2>(kv.first) << " were never waited for";
                return fail(os.str());
            }
        for (auto &kv : localInflight)
            if (!kv.second.empty()) {
                std::ostringstream os;
                os << "chunk " << ci << ": rank " << std::get<0>(kv.first) << " queue " << std::get<2>(kv.first) << " posted " << kv.second.size()
                   << " local notify(s) to queue " << std::get<1>(kv.first) << " that were never waited for";
                return fail(os.str());
            }
        // memory conflicts (user INPUT / OUTPUT of different ranks never alias; the same rank's INPUT and OUTPUT are
        // distinct buffers in the checked calls)
        std::sort(accesses.begin(), accesses.end(), [](const Access &a, const Access &b) { return std::tie(a.rank, a.kind, a.lo) < std::tie(b.rank, b.kind, b.lo); });
        for (size_t i = 0; i < accesses.size(); ++i) {
            for (size_t j = i + 1; j < accesses.size(); ++j) {
                const Access &a = accesses[i], &b = accesses[j];
                if (a.rank != b.rank || a.kind != b.kind || b.lo >= a.hi) break;
                if (!a.write && !b.write) continue;
                if (a.byRank == b.byRank && a.byQueue == b.byQueue) continue;            // program order
                if (HappensBefore(a.clock, b.clock) || HappensBefore(b.clock, a.clock)) continue;
                std::ostringstream os;
                os << "memory conflict in chunk " << ci << " on rank " << a.rank << " buffer kind " << a.kind << " bytes [" << std::max(a.lo, b.lo) << ", " << std::min(a.hi, b.hi)
                   << "): task " << a.taskIdx << " of rank " << a.byRank << "/q" << a.byQueue << (a.write ? " (write)" : " (read)") << " and task " << b.taskIdx << " of rank " << b.byRank
                   << "/q" << b.byQueue << (b.write ? " (write)" : " (read)") << " are not ordered";
                return fail(os.str());
            }
        }
    }
    // semantics
    auto expect = [&](uint32_t rank, uint64_t outElem, Value want) -> bool {
        std::sort(want.begin(), want.end());
        return w.At(rank, (int)BufKind::OUTPUT, outElem) == want;
    };
    auto bad = [&](uint32_t rank, uint64_t e) {
        std::ostringstream os;
        os << "semantic error: output element " << e << " of rank " << rank << " holds {";
        for (auto &c : w.At(rank, (int)BufKind::OUTPUT, e)) os << "(" << c.first << "," << c.second << ")";
        os << "}";
        return fail(os.str());
    };
    const uint64_t cnt = spec.count;
    for (uint32_t r = 0; r < n; ++r) {
        switch (spec.op) {
            case HCCL_CMD_ALLREDUCE:
                for (uint64_t i = 0; i < cnt; ++i) { Value v; for (uint32_t s = 0; s < n; ++s) v.push_back({s, i}); if (!expect(r, i, v)) return bad(r, i); }
                break;
            case HCCL_CMD_REDUCE:
                if (r == spec.root) for (uint64_t i = 0; i < cnt; ++i) { Value v; for (uint32_t s = 0; s < n; ++s) v.push_back({s, i}); if (!expect(r, i, v)) return bad(r, i); }
                break;
            case HCCL_CMD_ALLGATHER:
                for (uint32_t s = 0; s < n; ++s) for (uint64_t i = 0; i < cnt; ++i) if (!expect(r, s * cnt + i, {{s, i}})) return bad(r, s * cnt + i);
                break;
            case HCCL_CMD_REDUCE_SCATTER:
                for (uint64_t i = 0; i < cnt; ++i) { Value v; for (uint32_t s = 0; s < n; ++s) v.push_back({s, r * cnt + i}); if (!expect(r, i, v)) return bad(r, i); }
                break;
            case HCCL_CMD_BROADCAST:
                for (uint64_t i = 0; i < cnt; ++i) if (!expect(r, i, {{spec.root, i}})) return bad(r, i);
                break;
            case HCCL_CMD_SCATTER:
                for (uint64_t i = 0; i < cnt; ++i) if (!expect(r, i, {{spec.root, r * cnt + i}})) return bad(r, i);
                break;
            case HCCL_CMD_ALLTOALL:
                for (uint32_t s = 0; s < n; ++s) for (uint64_t i = 0; i < cnt; ++i) if (!expect(r, s * cnt + i, {{s, r * cnt + i}})) return bad(r, s * cnt + i);
                break;
            case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: {
                uint64_t ro = 0;
                for (uint32_t s = 0; s < n; ++s) {
                    uint64_t so = 0;
                    for (uint32_t j = 0; j < r; ++j) so += spec.countMatrix[s * n + j];
                    for (uint64_t i = 0; i < spec.countMatrix[s * n + r]; ++i) if (!expect(r, ro + i, {{s, so + i}})) return bad(r, ro + i);
                    ro += spec.countMatrix[s * n + r];
                }
                break;
            }
            case HCCL_CMD_ALLGATHER_V: {
                uint64_t o = 0;
                for (uint32_t s = 0; s < n; ++s) { for (uint64_t i = 0; i < spec.countMatrix[s]; ++i) if (!expect(r, o + i, {{s, i}})) return bad(r, o + i); o += spec.countMatrix[s]; }
                break;
            }
            case HCCL_CMD_REDUCE_SCATTER_V: {
                uint64_t o = 0;
                for (uint32_t j = 0; j < r; ++j) o += spec.countMatrix[j];
                for (uint64_t i = 0; i < spec.countMatrix[r]; ++i) { Value v; for (uint32_t s = 0; s < n; ++s) v.push_back({s, o + i}); if (!expect(r, i, v)) return bad(r, i); }
                break;
            }
            case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE:
                if (r == spec.peer) for (uint64_t i = 0; i < cnt; ++i) if (!expect(r, i, {{spec.root, i}})) return bad(r, i);
                break;
            case HCCL_CMD_BATCH_SEND_RECV: {
                // first half arrives from rank - 1, second half from rank + 1 (their matching halves)
                const uint64_t h = cnt / 2;
                const uint32_t prev = (r + n - 1) % n, next = (r + 1) % n;
                for (uint64_t i = 0; i < h; ++i) if (!expect(r, i, {{prev, i}})) return bad(r, i);
                for (uint64_t i = h; i < cnt; ++i) if (!expect(r, i, {{next, i}})) return bad(r, i);
                break;
            }
            default: break;   // barrier: deadlock / notify balance only
        }
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
