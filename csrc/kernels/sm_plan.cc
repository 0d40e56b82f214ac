#include <algorithm>
#include <functional>
#include "../common/dtype.h"
#include "../common/log.h"
#include "coll_args.h"

namespace hccl {

namespace {
uint64_t Down128(uint64_t v) { return v & ~127ull; }
uint64_t Up128(uint64_t v) { return (v + 127) & ~127ull; }
uint64_t Clamp(uint64_t total, uint64_t lo, uint64_t chunk) { return total <= lo ? 0 : std::min(chunk, total - lo); }
}  // namespace

// Enough CTAs to keep NVLink busy (about 1 MB in flight at 512 threads x 4 x 16 B per CTA), few for small payloads
// where launch and flag latency dominate.
uint32_t SmCtasFor(uint64_t bytes, uint32_t maxCtas)
{
    uint32_t c;
    if (bytes <= (16u << 10)) c = 1;
    else if (bytes <= (64u << 10)) c = 4;
    else if (bytes <= (256u << 10)) c = 8;
    else if (bytes <= (1u << 20)) c = 16;
    else if (bytes <= (4u << 20)) c = 32;
    else if (bytes <= (32u << 20)) c = 64;
    else c = 96;
    if (maxCtas) c = std::min(c, maxCtas);
    return std::max(1u, std::min<uint32_t>(c, kMaxChannels));
}

HcclResult SmPlanOp(const SmPlanCtx &ctx, const OpParam &p, const std::string &alg, std::vector<SmLaunch> *out)
{
    const uint32_t n = ctx.nranks, me = ctx.rank;
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t ccl = ctx.cclBytes;
    SmLaunch base{};
    base.dtype = p.dtype;
    base.args.elemSize = es;
    base.args.root = p.root;
    base.args.op = (uint32_t)p.reduceOp;
    base.args.peer = p.peer;

    // chunk loop: calls emit(lo, n) for element ranges of at most maxCount
    auto loop = [&](uint64_t total, uint64_t maxCount, const std::function<void(uint64_t, uint64_t)> &emit) -> HcclResult {
        if (maxCount == 0) { HCCL_ERROR("%s: CCL buffer of %llu bytes is too small for %u ranks", alg.c_str(), (unsigned long long)ccl, n); return HCCL_E_MEMORY; }
        for (uint64_t lo = 0; lo < total; lo += maxCount) emit(lo, std::min(maxCount, total - lo));
        return HCCL_SUCCESS;
    };
    auto push = [&](SmKernelId k, uint64_t lo, uint64_t cnt, uint64_t ctaBytes, const std::function<void(SmLaunch &)> &fill) {
        SmLaunch l = base;
        l.kernel = k;
        l.args.count = cnt;
        l.args.bytes = cnt * es;
        l.ctas = SmCtasFor(ctaBytes, ctx.maxCtas);
        (void)lo;
        fill(l);
        out->push_back(l);
    };
    const char *in = (const char *)p.inputPtr;
    char *outp = (char *)p.outputPtr;

    if (alg == "SmAllReduceMesh1DOneShot" || alg == "NvlsAllReduceOneShot") {
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        uint64_t maxCount = nv ? Down128(ccl) / es : Down128(ccl / n) / es;
        return loop(p.count, maxCount, [&](uint64_t lo, uint64_t cnt) {
            push(nv ? K_ALLREDUCE_NVLS_ONESHOT : K_ALLREDUCE_ONESHOT, lo, cnt, cnt * es, [&](SmLaunch &l) { l.args.in = in + lo * es; l.args.out = outp + lo * es; });
        });
    }
    if (alg == "SmAllReduceMesh1DTwoShot" || alg == "NvlsAllReduceTwoShot") {
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        uint64_t maxSlice = Down128(ccl / (nv ? 2 * n : n + 1));
        uint64_t maxCount = maxSlice * n / es;
        return loop(p.count, maxCount, [&](uint64_t lo, uint64_t cnt) {
            push(nv ? K_ALLREDUCE_NVLS_TWOSHOT : K_ALLREDUCE_TWOSHOT, lo, cnt, cnt * es / n * 2, [&](SmLaunch &l) { l.args.in = in + lo * es; l.args.out = outp + lo * es; });
        });
    }
    if (alg == "SmAllReduceConcurrent" || alg == "NvlsAllReduceConcurrent") {
        // One payload, two algorithms side by side in one launch. Shares come from HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO
        // ("a:b"); unset, the switch-reduced part gets two thirds (it moves a third of the bytes of the peer-store part
        // into each GPU), and an even split when both parts use peer stores.
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        uint32_t ra = ctx.splitRatio[0], rb = ctx.splitRatio[1];
        if (ra + rb == 0) { ra = nv ? 2 : 1; rb = 1; }
        if (ccl < 4ull * n * 128 + 4096) return HCCL_E_MEMORY;
        // scratch: part A up to 2 n slices, part B n + 1 slices; 2 * (bytes + n * 128) covers both
        uint64_t maxBytes = Down128(ccl / 2) - (uint64_t)n * 256;
        uint64_t unit = (uint64_t)n * 128;                         // part A stays a whole number of aligned slices
        uint64_t maxCount = maxBytes / unit * unit / es;
        if (maxCount == 0) return HCCL_E_MEMORY;
        return loop(p.count, maxCount, [&](uint64_t lo, uint64_t cnt) {
            uint64_t bytes = cnt * es;
            uint64_t a = bytes * ra / (ra + rb) / unit * unit;
            if (rb == 0) a = bytes;
            push(nv ? K_ALLREDUCE_CONCURRENT_NVLS : K_ALLREDUCE_CONCURRENT, lo, cnt, cnt * es / n * 2, [&](SmLaunch &l) {
                l.args.in = in + lo * es; l.args.out = outp + lo * es;
                l.ctas = std::max(2u, l.ctas);
                l.args.splitBytes = a;
                uint32_t ca = (uint32_t)((uint64_t)l.ctas * ra / (ra + rb));
                l.args.splitCtas = std::min(l.ctas - 1, std::max(1u, ca));
            });
        });
    }
    if (alg.size() > 8 && alg.compare(alg.size() - 8, 8, "ZeroCopy") == 0) {
        // Registered windows on both sides of the transfer that crosses ranks; one launch for any size (no scratch, no chunks).
        const bool nv = alg[0] == 'N';
        if (nv && !ctx.nvls) return HCCL_E_NOT_SUPPORT;
        if (!ctx.registeredOffset) return HCCL_E_NOT_SUPPORT;
        const uint64_t bytes = p.count * es;
        if (bytes == 0 || bytes % 16 || ((uintptr_t)in & 15u) || ((uintptr_t)outp & 15u)) return HCCL_E_NOT_SUPPORT;
        uint64_t inOff = 0, outOff = 0;
        SmKernelId id;
        uint64_t moved = bytes;
        if (p.opType == HCCL_CMD_ALLREDUCE) {
            if (!ctx.registeredOffset(in, bytes, &inOff) || !ctx.registeredOffset(outp, bytes, &outOff)) return HCCL_E_NOT_SUPPORT;
            id = nv ? K_ALLREDUCE_ZC_NVLS : K_ALLREDUCE_ZC;
            moved = bytes / n * 2;
        } else if (p.opType == HCCL_CMD_REDUCE_SCATTER) {
            if (!ctx.registeredOffset(in, bytes * n, &inOff)) return HCCL_E_NOT_SUPPORT;
            id = nv ? K_REDUCESCATTER_ZC_NVLS : K_REDUCESCATTER_ZC;
        } else if (p.opType == HCCL_CMD_ALLGATHER) {
            if (!ctx.registeredOffset(outp, bytes * n, &outOff)) return HCCL_E_NOT_SUPPORT;
            id = nv ? K_ALLGATHER_ZC_NVLS : K_ALLGATHER_ZC;
            moved = bytes * (n - 1);
        } else if (p.opType == HCCL_CMD_BROADCAST) {
            if (!ctx.registeredOffset(outp, bytes, &outOff)) return HCCL_E_NOT_SUPPORT;
            id = nv ? K_BROADCAST_ZC_NVLS : K_BROADCAST_ZC;
        } else return HCCL_E_NOT_SUPPORT;
        push(id, 0, p.count, moved, [&](SmLaunch &l) { l.args.in = in; l.args.out = outp; l.args.inOff = inOff; l.args.outOff = outOff; });
        return HCCL_SUCCESS;
    }
    if (alg == "SmAllReduceRing") {
        if (n < 2) return HCCL_E_NOT_SUPPORT;
        uint64_t maxSlice = Down128(ccl / (2 * (n - 1)));
        uint64_t maxCount = maxSlice * n / es;
        return loop(p.count, maxCount, [&](uint64_t lo, uint64_t cnt) {
            push(K_ALLREDUCE_RING, lo, cnt, cnt * es / n * 2, [&](SmLaunch &l) { l.args.in = in + lo * es; l.args.out = outp + lo * es; });
        });
    }
    // ---- warp-specialised pipelines: one launch for any payload; the scratch half holds rings of sub-chunks
    auto pipeSub = [&](uint32_t rings, uint32_t ctas) -> uint64_t {
        uint64_t s = Down128(ccl / ((uint64_t)rings * 2 /* depth */ * n * ctas));
        return std::min<uint64_t>(s, 256u << 10);
    };
    auto pipeCtas = [&](uint64_t movedBytes) { return std::min<uint32_t>(SmCtasFor(movedBytes, ctx.maxCtas), kPipeChannels); };
    if (alg == "SmAllReducePipelined" || alg == "NvlsAllReducePipelined") {
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        SmLaunch l = base;
        l.kernel = nv ? K_ALLREDUCE_PIPE_NVLS : K_ALLREDUCE_PIPE;
        l.args.count = p.count; l.args.bytes = p.count * es; l.args.in = in; l.args.out = outp;
        l.ctas = pipeCtas(p.count * es / n * 2);
        l.args.pipeSub = pipeSub(2, l.ctas);
        if (l.args.pipeSub < 128) return HCCL_E_NOT_SUPPORT;
        out->push_back(l);
        return HCCL_SUCCESS;
    }
    if (alg == "SmReduceScatterPipelined" || alg == "SmReduceScatterVPipelined" || alg == "NvlsReduceScatterPipelined") {
        bool v = p.opType == HCCL_CMD_REDUCE_SCATTER_V;
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || v || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        uint64_t longest = v ? *std::max_element(p.sendCounts.begin(), p.sendCounts.end()) : p.count;
        SmLaunch l = base;
        l.kernel = nv ? K_REDUCESCATTER_PIPE_NVLS : K_REDUCESCATTER_PIPE;
        l.args.in = in; l.args.out = outp;
        for (uint32_t r = 0; r < n; ++r) {
            l.args.sendBytes[r] = (v ? p.sendCounts[r] : p.count) * es;
            l.args.sendOff[r] = (v ? p.sendDispls[r] : (uint64_t)r * p.count) * es;
        }
        l.ctas = pipeCtas(longest * es * (n - 1));
        l.args.pipeSub = pipeSub(1, l.ctas);
        if (l.args.pipeSub < 128) return HCCL_E_NOT_SUPPORT;
        out->push_back(l);
        return HCCL_SUCCESS;
    }
    if (alg == "SmAllGatherPush" || alg == "SmAllGatherVPush" || alg == "NvlsAllGatherPush" || alg == "NvlsAllGatherVPush") {
        bool v = p.opType == HCCL_CMD_ALLGATHER_V;
        bool nv = alg[0] == 'N';
        if (nv && !ctx.nvls) return HCCL_E_NOT_SUPPORT;
        uint64_t longest = v ? *std::max_element(p.recvCounts.begin(), p.recvCounts.end()) : p.count;
        SmLaunch l = base;
        l.kernel = nv ? K_ALLGATHER_PIPE_NVLS : K_ALLGATHER_PIPE;
        l.args.in = in; l.args.out = outp;
        for (uint32_t r = 0; r < n; ++r) {
            l.args.recvBytes[r] = (v ? p.recvCounts[r] : p.count) * es;
            l.args.recvOff[r] = (v ? p.recvDispls[r] : (uint64_t)r * p.count) * es;
        }
        l.ctas = pipeCtas(longest * es * (n - 1));
        l.args.pipeSub = pipeSub(1, l.ctas);
        if (l.args.pipeSub < 128) return HCCL_E_NOT_SUPPORT;
        out->push_back(l);
        return HCCL_SUCCESS;
    }
    // Broadcast as a one-contributor push: only the root owns a (non-empty) piece, everybody drains slot `root`.
    if (alg == "SmBroadcastPush" || alg == "NvlsBroadcastPush") {
        bool nv = alg[0] == 'N';
        if (nv && !ctx.nvls) return HCCL_E_NOT_SUPPORT;
        SmLaunch l = base;
        l.kernel = nv ? K_ALLGATHER_PIPE_NVLS : K_ALLGATHER_PIPE;
        l.args.in = outp; l.args.out = outp;
        for (uint32_t r = 0; r < n; ++r) { l.args.recvBytes[r] = r == p.root ? p.count * es : 0; l.args.recvOff[r] = 0; }
        if (me != p.root) l.args.in = nullptr;
        l.ctas = pipeCtas(p.count * es);
        l.args.pipeSub = pipeSub(1, l.ctas);
        if (l.args.pipeSub < 128) return HCCL_E_NOT_SUPPORT;
        out->push_back(l);
        return HCCL_SUCCESS;
    }
    if (alg == "SmAlltoAllPush") {
        SmLaunch l = base;
        l.kernel = K_ALLTOALL_PIPE;
        l.args.in = in; l.args.out = outp;
        for (uint32_t r = 0; r < n; ++r) {
            l.args.sendBytes[r] = l.args.recvBytes[r] = p.count * es;
            l.args.sendOff[r] = l.args.recvOff[r] = (uint64_t)r * p.count * es;
        }
        l.ctas = pipeCtas(p.count * es * (n - 1));
        l.args.pipeSub = pipeSub(1, l.ctas);
        if (l.args.pipeSub < 128) return HCCL_E_NOT_SUPPORT;
        out->push_back(l);
        return HCCL_SUCCESS;
    }
    if (alg == "SmAllGatherMesh1D" || alg == "SmAllGatherVMesh1D") {
        bool v = p.opType == HCCL_CMD_ALLGATHER_V;
        uint64_t total = v ? *std::max_element(p.recvCounts.begin(), p.recvCounts.end()) : p.count;
        return loop(total, Down128(ccl) / es, [&](uint64_t lo, uint64_t cnt) {
            // from 128 KB per rank the pull is short of requests in flight with the generic CTA count (16 CTAs at 256 KB x 3 peers
            // measured 21.7 us against 14.5 us for the 1 KB floor): size the grid as for four times the bytes
            push(K_ALLGATHER_V, lo, cnt, cnt * es * (n - 1) * (cnt * es >= (128u << 10) ? 4 : 1), [&](SmLaunch &l) {
                l.args.in = in + lo * es;
                l.args.out = outp;
                for (uint32_t r = 0; r < n; ++r) {
                    l.args.recvBytes[r] = (v ? Clamp(p.recvCounts[r], lo, cnt) : cnt) * es;
                    l.args.recvOff[r] = ((v ? p.recvDispls[r] : (uint64_t)r * p.count) + lo) * es;
                }
            });
        });
    }
    if (alg == "SmReduceScatterMesh1D" || alg == "SmReduceScatterVMesh1D" || alg == "NvlsReduceScatter") {
        bool v = p.opType == HCCL_CMD_REDUCE_SCATTER_V;
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || v || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        uint64_t total = v ? *std::max_element(p.sendCounts.begin(), p.sendCounts.end()) : p.count;
        return loop(total, Down128(ccl / n) / es, [&](uint64_t lo, uint64_t cnt) {
            push(nv ? K_REDUCESCATTER_NVLS : K_REDUCESCATTER_V, lo, cnt, cnt * es * (n - 1), [&](SmLaunch &l) {
                l.args.in = in;
                l.args.out = outp + lo * es;
                for (uint32_t r = 0; r < n; ++r) {
                    l.args.sendBytes[r] = (v ? Clamp(p.sendCounts[r], lo, cnt) : cnt) * es;
                    l.args.sendOff[r] = ((v ? p.sendDispls[r] : (uint64_t)r * p.count) + lo) * es;
                }
            });
        });
    }
    if (alg == "SmBroadcastMesh1D" || alg == "NvlsBroadcast") {
        bool nv = alg[0] == 'N';
        if (nv && (!ctx.nvls || (p.count * es) % 16 != 0)) return HCCL_E_NOT_SUPPORT;
        return loop(p.count, Down128(ccl) / es, [&](uint64_t lo, uint64_t cnt) {
            push(nv ? K_BROADCAST_NVLS : K_BROADCAST, lo, cnt, cnt * es, [&](SmLaunch &l) { l.args.in = outp + lo * es; l.args.out = outp + lo * es; });
        });
    }
    if (alg == "SmReduceMesh1D") {
        return loop(p.count, Down128(ccl / n) / es, [&](uint64_t lo, uint64_t cnt) {
            push(K_REDUCE, lo, cnt, cnt * es, [&](SmLaunch &l) { l.args.in = in + lo * es; l.args.out = outp ? outp + lo * es : nullptr; });
        });
    }
    if (alg == "SmScatterMesh1D") {
        return loop(p.count, Down128(ccl / n) / es, [&](uint64_t lo, uint64_t cnt) {
            push(K_SCATTER, lo, cnt, cnt * es, [&](SmLaunch &l) {
                l.args.in = in;
                l.args.out = outp + lo * es;
                for (uint32_t r = 0; r < n; ++r) { l.args.sendBytes[r] = cnt * es; l.args.sendOff[r] = ((uint64_t)r * p.count + lo) * es; }
            });
        });
    }
    if (alg == "SmAlltoAllMesh1D" || alg == "SmAlltoAllVMesh1D" || alg == "SmAlltoAllVCMesh1D") {
        // One launch for any payload: a pair longer than its scratch slot moves in rounds inside the kernel. The slot size and
        // the grid are functions of the communicator only, so they agree on every rank whatever the count matrix is.
        const bool fixed = alg == "SmAlltoAllMesh1D";
        const uint32_t esOut = fixed ? es : DataTypeSize(p.outDtype);
        const uint64_t usable = ccl > kA2aMetaBytes ? ccl - kA2aMetaBytes : 0;
        const uint64_t slot = n > 1 ? Down128(usable / (n - 1)) : Down128(usable);
        if (slot < 128) { HCCL_ERROR("AlltoAll: a CCL buffer of %llu bytes leaves no scratch slot per peer (%u ranks)", (unsigned long long)ccl, n); return HCCL_E_MEMORY; }
        push(K_ALLTOALL_V, 0, fixed ? p.count : 0, fixed ? p.count * es * (n - 1) : 0, [&](SmLaunch &l) {
            // the grid must be the same on every rank (channels synchronise pairwise across ranks), so the variable forms
            // cannot size it from this rank's own counts
            if (!fixed) l.ctas = ctx.maxCtas ? std::min(16u, ctx.maxCtas) : 16u;
            l.args.in = in;
            l.args.out = outp;
            l.args.slotBytes = slot;
            for (uint32_t r = 0; r < n; ++r) {
                if (fixed) {
                    l.args.sendBytes[r] = l.args.recvBytes[r] = p.count * es;
                    l.args.sendOff[r] = l.args.recvOff[r] = (uint64_t)r * p.count * es;
                } else {
                    l.args.sendBytes[r] = p.sendCounts[r] * es; l.args.sendOff[r] = p.sendDispls[r] * es;
                    l.args.recvBytes[r] = p.recvCounts[r] * esOut; l.args.recvOff[r] = p.recvDispls[r] * esOut;
                }
            }
        });
        return HCCL_SUCCESS;
    }
    if (alg == "SmBarrierMesh1D") {
        push(K_BARRIER, 0, 0, 0, [&](SmLaunch &) {});
        return HCCL_SUCCESS;
    }
    if (alg == "SmSend" || alg == "SmRecv") {
        bool snd = alg == "SmSend";
        push(snd ? K_SEND : K_RECV, 0, p.count, 0, [&](SmLaunch &l) { l.args.in = in; l.args.out = outp; l.ctas = kP2pBlocks; });
        return HCCL_SUCCESS;
    }
    if (alg == "SmBatchSendRecv") {
        // queue per (peer, direction); self pairs become local copies. Same ordering rules as the host engine.
        std::vector<HcclSendRecvItem> sends, recvs, selfS, selfR;
        for (auto &it : p.items) {
            if (it.remoteRank == me) (it.sendRecvType == HCCL_SEND ? selfS : selfR).push_back(it);
            else (it.sendRecvType == HCCL_SEND ? sends : recvs).push_back(it);
        }
        if (selfS.size() != selfR.size()) return HCCL_E_PARA;
        if (p.items.size() > (size_t)kMaxBatchItems) return HCCL_E_NOT_SUPPORT;   // the host-issued engine takes large batches
        SmLaunch l = base;
        l.kernel = K_BATCH_SEND_RECV;
        BatchArgs &b = l.batch;
        b.nItems = 0;
        std::vector<std::pair<uint32_t, uint32_t>> queues;   // (peer, dir)
        auto queueOf = [&](uint32_t peer, uint32_t dir) {
            for (size_t q = 0; q < queues.size(); ++q) if (queues[q] == std::make_pair(peer, dir)) return (uint32_t)q;
            queues.push_back({peer, dir});
            return (uint32_t)queues.size() - 1;
        };
        std::vector<uint32_t> orderInQueue;
        auto add = [&](const HcclSendRecvItem &it, uint32_t isSend) {
            BatchItem &bi = b.items[b.nItems++];
            bi.buf = it.buf; bi.bytes = it.count * DataTypeSize(it.dataType); bi.peer = it.remoteRank; bi.isSend = isSend; bi.buf2 = nullptr;
            bi.queue = queueOf(it.remoteRank, isSend);
            if (orderInQueue.size() <= bi.queue) orderInQueue.resize(bi.queue + 1, 0);
            bi.order = orderInQueue[bi.queue]++;
        };
        for (auto &it : sends) add(it, 1);
        for (auto &it : recvs) add(it, 0);
        for (size_t i = 0; i < selfS.size(); ++i) {
            uint64_t sb = selfS[i].count * DataTypeSize(selfS[i].dataType), rb = selfR[i].count * DataTypeSize(selfR[i].dataType);
            if (sb != rb) return HCCL_E_PARA;
            BatchItem &bi = b.items[b.nItems++];
            bi.buf = selfS[i].buf; bi.buf2 = selfR[i].buf; bi.bytes = sb; bi.peer = me; bi.isSend = 2;
            bi.queue = queueOf(me, 2 + (uint32_t)i);
            bi.order = 0;
        }
        b.nQueues = (uint32_t)queues.size();
        l.ctas = b.nQueues * kP2pBlocks;
        if (l.ctas > (uint32_t)kMaxChannels) return HCCL_E_NOT_SUPPORT;
        out->push_back(l);
        return HCCL_SUCCESS;
    }
    HCCL_ERROR("unknown SM algorithm %s", alg.c_str());
    return HCCL_E_NOT_FOUND;
}

}  // namespace hccl
