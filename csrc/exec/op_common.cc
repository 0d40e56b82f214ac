#include "../common/launch_count.h"
#include "op_common.h"
#include <algorithm>
#include <atomic>
#include <unordered_map>
#include "../kernels/coll_args.h"
#include "../kernels/launch.h"
#include <chrono>
#include <cstring>
#include "../common/dtype.h"
#include "../common/log.h"
#include "../select/selector.h"
#include "executor.h"

namespace hccl {

void EnsureSelectorsLinked();
extern bool CudaStreamIsCapturing(cudaStream_t s);
extern HcclResult CudaMemcpyAsyncD2D(void *dst, const void *src, uint64_t bytes, cudaStream_t s);
extern void NvtxPush(const char *name);
extern void NvtxPop();

static uint64_t NowNs()
{
    using namespace std::chrono;
    return (uint64_t)duration_cast<nanoseconds>(steady_clock::now().time_since_epoch()).count();
}

bool StreamIsCapturing(cudaStream_t s) { return CudaStreamIsCapturing(s); }

HcclResult LocalCopyAsync(Comm *c, void *dst, const void *src, uint64_t bytes, cudaStream_t s)
{
    if (bytes == 0 || dst == src) return HCCL_SUCCESS;
    if (c->backend == BackendKind::SIM) {
        c->worker->Enqueue([dst, src, bytes] { memmove(dst, src, bytes); return HCCL_SUCCESS; });
        return HCCL_SUCCESS;
    }
    return CudaMemcpyAsyncD2D(dst, src, bytes, s);
}

HcclResult SingleRankProc(Comm *c, OpParam &p)
{
    uint64_t es = DataTypeSize(p.dtype);
    switch (p.opType) {
        case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE:
            HCCL_WARNING("%s on a single-rank communicator is a no-op", CmdName(p.opType));
            return HCCL_SUCCESS;
        case HCCL_CMD_BROADCAST: case HCCL_CMD_BARRIER: return HCCL_SUCCESS;
        case HCCL_CMD_BATCH_SEND_RECV: {
            // only self pairs can exist
            std::vector<HcclSendRecvItem> s, r;
            for (auto &it : p.items) (it.sendRecvType == HCCL_SEND ? s : r).push_back(it);
            if (s.size() != r.size()) return HCCL_E_PARA;
            for (size_t i = 0; i < s.size(); ++i) CHK_RET(LocalCopyAsync(c, r[i].buf, s[i].buf, s[i].count * DataTypeSize(s[i].dataType), p.stream));
            return HCCL_SUCCESS;
        }
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
            return LocalCopyAsync(c, (char *)p.outputPtr + p.recvDispls[0] * DataTypeSize(p.outDtype),
                                  (const char *)p.inputPtr + p.sendDispls[0] * es, p.sendCounts[0] * es, p.stream);
        case HCCL_CMD_ALLGATHER_V:
            return LocalCopyAsync(c, (char *)p.outputPtr + p.recvDispls[0] * es, p.inputPtr, p.count * es, p.stream);
        case HCCL_CMD_REDUCE_SCATTER_V:
            return LocalCopyAsync(c, p.outputPtr, (const char *)p.inputPtr + p.sendDispls[0] * es, p.count * es, p.stream);
        default: return LocalCopyAsync(c, p.outputPtr, p.inputPtr, p.count * es, p.stream);
    }
}

HcclResult SelectAlgorithm(Comm *c, OpParam &p, const std::vector<HcclCommEngine> &excluded)
{
    EnsureSelectorsLinked();
    SelectorCtx ctx;
    ctx.comm = c;
    ctx.topo = &c->topo;
    ctx.env = &c->env;
    ctx.cuda = c->backend == BackendKind::CUDA;
    ctx.nvls = c->mcHeap != nullptr;
    ctx.cclBytes = c->devComm.cclBytes;
    ctx.excluded = excluded;
    CHK_RET(ExecuteSelector(ctx, p));
    p.algTag = p.tag + "_" + p.algName + "_" + EngineName(p.engine);
    p.execTimeoutSec = c->env.execTimeoutSec;
    return HCCL_SUCCESS;
}

void FillOpExchangeInfo(Comm *c, const OpParam &p, OpExchangeInfo *info)
{
    memset(info, 0, sizeof(*info));
    info->cclBufferSize = c->devComm.cclBytes;
    info->root = p.root;
    info->opType = (uint32_t)p.opType;
    info->engine = (uint32_t)p.engine;
    info->reduceOp = (uint32_t)p.reduceOp;
    info->dataType = (uint32_t)p.dtype;
    info->count = p.count;
    info->ctaLimit = c->env.maxCtas;
    snprintf(info->group, sizeof(info->group), "%s", c->name.c_str());
    snprintf(info->algName, sizeof(info->algName), "%s", p.algName.c_str());
    snprintf(info->tag, sizeof(info->tag), "%s", p.tag.c_str());
}

HcclResult CompareOpExchangeInfos(const std::vector<OpExchangeInfo> &all, uint32_t myRank, std::string *why)
{
    const OpExchangeInfo &me = all[myRank];
    auto hasRoot = [](uint32_t op) { return op == HCCL_CMD_BROADCAST || op == HCCL_CMD_REDUCE || op == HCCL_CMD_SCATTER; };
    auto hasReduce = [](uint32_t op) { return op == HCCL_CMD_ALLREDUCE || op == HCCL_CMD_REDUCE || op == HCCL_CMD_REDUCE_SCATTER || op == HCCL_CMD_REDUCE_SCATTER_V; };
    auto varCount = [](uint32_t op) { return op == HCCL_CMD_ALLTOALLV || op == HCCL_CMD_ALLTOALLVC || op == HCCL_CMD_ALLGATHER_V || op == HCCL_CMD_REDUCE_SCATTER_V || op == HCCL_CMD_BARRIER; };
    for (uint32_t r = 0; r < all.size(); ++r) {
        if (r == myRank) continue;
        const OpExchangeInfo &o = all[r];
        char buf[512];
#define MISMATCH(field, fmt, a, b)                                                                                       \
    do {                                                                                                                 \
        snprintf(buf, sizeof(buf), "[EI0005] %s differs between rank %u (" fmt ") and rank %u (" fmt ") for tag %s", field, myRank, a, r, b, me.tag); \
        if (why) *why = buf;                                                                                             \
        return HCCL_E_PARA;                                                                                              \
    } while (0)
        if (me.opType != o.opType) MISMATCH("opType", "%u", me.opType, o.opType);
        if (strncmp(me.tag, o.tag, sizeof(me.tag)) != 0) MISMATCH("tag", "%s", me.tag, o.tag);
        if (me.dataType != o.dataType) MISMATCH("dataType", "%u", me.dataType, o.dataType);
        if (!varCount(me.opType) && me.count != o.count) MISMATCH("count", "%llu", (unsigned long long)me.count, (unsigned long long)o.count);
        if (hasReduce(me.opType) && me.reduceOp != o.reduceOp) MISMATCH("reduceOp", "%u", me.reduceOp, o.reduceOp);
        if (hasRoot(me.opType) && me.root != o.root) MISMATCH("root", "%u", me.root, o.root);
        if (me.cclBufferSize != o.cclBufferSize) MISMATCH("cclBufferSize", "%llu", (unsigned long long)me.cclBufferSize, (unsigned long long)o.cclBufferSize);
        if (me.engine != o.engine) MISMATCH("engine", "%u", me.engine, o.engine);
        if (strncmp(me.algName, o.algName, sizeof(me.algName)) != 0) MISMATCH("algName", "%s", me.algName, o.algName);
        if (me.ctaLimit != o.ctaLimit) MISMATCH("ctaLimit", "%u", me.ctaLimit, o.ctaLimit);
#undef MISMATCH
    }
    return HCCL_SUCCESS;
}

HcclResult CheckOpConsistency(Comm *c, const OpParam &p)
{
    if (c->env.inconsistentCheck == InconsistentCheck::OFF) return HCCL_SUCCESS;
    if (p.opType == HCCL_CMD_SEND || p.opType == HCCL_CMD_RECEIVE || p.opType == HCCL_CMD_BATCH_SEND_RECV) return HCCL_SUCCESS;
    if (p.mode == OpMode::OFFLOAD || (c->backend == BackendKind::CUDA && StreamIsCapturing(p.stream))) return HCCL_SUCCESS;
    std::string key = p.algTag + "|" + std::to_string((int)p.dtype) + "|" + std::to_string((int)p.reduceOp);
    if (c->env.inconsistentCheck == InconsistentCheck::FIRST) {
        std::lock_guard<std::mutex> lk(c->ctxMu);
        if (c->consistencyDone.count(key)) return HCCL_SUCCESS;
        c->consistencyDone[key] = true;
    }
    OpExchangeInfo mine;
    FillOpExchangeInfo(c, p, &mine);
    std::vector<OpExchangeInfo> all(c->nranks);
    CHK_RET(c->boot->AllGather(&mine, sizeof(mine), all.data()));
    c->counters.consistencyChecks++;
    std::string why;
    HcclResult r = CompareOpExchangeInfos(all, c->rank, &why);
    if (r != HCCL_SUCCESS) HCCL_ERROR("%s", why.c_str());
    return r;
}

// ---- fast path: a call that repeats an earlier one (same operator, buffers, count, types) replays its launch list.
// Selection, consistency exchange, executor construction and planning are skipped; what remains is a hash lookup and
// the kernel launches. Entries die with the tuning table / environment generation they were made under.
namespace {
struct FastKey {
    uint32_t op, dtype, rop, root;
    uint64_t count;
    const void *in;
    void *out;
    bool operator==(const FastKey &o) const { return op == o.op && dtype == o.dtype && rop == o.rop && root == o.root && count == o.count && in == o.in && out == o.out; }
};
struct FastHash {
    size_t operator()(const FastKey &k) const
    {
        uint64_t h = 1469598103934665603ull;
        auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; };
        mix(k.op | ((uint64_t)k.dtype << 8) | ((uint64_t)k.rop << 16) | ((uint64_t)k.root << 24));
        mix(k.count); mix((uint64_t)(uintptr_t)k.in); mix((uint64_t)(uintptr_t)k.out);
        return (size_t)h;
    }
};
struct FastEntry {
    std::string algName;
    HcclCommEngine engine;
    std::vector<SmLaunch> launches;
    uint64_t generation;
    uint64_t *histogramSlot;
    uint64_t lastUse;
};
struct FastCache { std::unordered_map<FastKey, FastEntry, FastHash> map; uint64_t tick = 0; };
constexpr size_t kFastCacheCap = 8192;
std::atomic<uint64_t> g_selectGeneration{1};

bool FastEligible(const Comm *c, const OpParam &p)
{
    static const bool enabled = [] { const char *e = getenv("HCCL_FAST_DISPATCH"); return e ? atoi(e) != 0 : true; }();
    if (!enabled) return false;
    if (c->backend != BackendKind::CUDA || p.mode != OpMode::OPBASE || c->env.entryLogEnable) return false;
    if (c->env.inconsistentCheck == InconsistentCheck::EVERY) return false;     // every call is cross-checked in that mode
    if (!p.sendCounts.empty() || !p.recvCounts.empty() || !p.items.empty()) return false;
    switch (p.opType) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_ALLGATHER: case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_BROADCAST: case HCCL_CMD_REDUCE:
        case HCCL_CMD_SCATTER: case HCCL_CMD_ALLTOALL: case HCCL_CMD_BARRIER: return true;
        default: return false;
    }
}
}  // namespace

void BumpSelectionGeneration() { g_selectGeneration.fetch_add(1); }

HcclResult HcclExecOp(Comm *c, OpParam &p)
{
    uint64_t begin = NowNs();
    CHK_RET(CommCheckReady(c));
    if (OpRetryEnabled(c) && !c->inRetry.load() && c->nranks > 1) RecordOpForRetry(c, p);
    // test hook: the operator goes through selection and the consistency exchange like any other, but is never launched here
    bool dropThisOp = false;
    if (c->injectOpDrop.load() > 0 && !c->inRetry.load() && c->nranks > 1) {
        c->injectOpDrop--;
        dropThisOp = true;
        HCCL_WARNING("comm %s rank %u: operator %s dropped by injection", c->name.c_str(), c->rank, CmdName(p.opType));
    }
    const bool fastOk = c->nranks > 1 && FastEligible(c, p);
    FastKey fkey{(uint32_t)p.opType, (uint32_t)p.dtype, (uint32_t)p.reduceOp, p.root, p.count, p.inputPtr, p.outputPtr};
    if (fastOk && c->fastOps && !dropThisOp) {
        auto *fc = static_cast<FastCache *>(c->fastOps.get());
        auto it = fc->map.find(fkey);
        if (it != fc->map.end() && it->second.generation == g_selectGeneration.load(std::memory_order_relaxed)) {
            FastEntry &e = it->second;
            e.lastUse = ++fc->tick;
            for (const SmLaunch &l : e.launches) {
                HcclResult lr = SmIssueLaunch(c->devCommPtr, l, p.stream);
                if (lr != HCCL_SUCCESS) return lr;
            }
            c->counters.kernelsLaunched += e.launches.size();
            const uint32_t devSeq = (uint32_t)c->devOpIssued.fetch_add(e.launches.size());
            CountLaunch(e.launches.size());
            c->counters.chunkLoops += e.launches.size();
            c->counters.planCacheHits++;
            OpRecord rec{};
            rec.seq = c->counters.ops++;
            rec.opType = p.opType; rec.dtype = p.dtype; rec.reduceOp = p.reduceOp; rec.count = p.count; rec.root = p.root; rec.engine = (uint32_t)e.engine;
            snprintf(rec.algName, sizeof(rec.algName), "%s", e.algName.c_str());
            rec.beginNs = begin;
            rec.endNs = NowNs();
            rec.devSeq = devSeq; rec.devLaunches = (uint32_t)e.launches.size();
            RecordOp(c, rec);
            c->counters.bytes += p.DataBytes();
            {
                std::lock_guard<std::mutex> lk(c->counters.mu);
                ++*e.histogramSlot;
            }
            return HCCL_SUCCESS;
        }
    }
    std::vector<SmLaunch> captured;
    struct CaptureScope {
        explicit CaptureScope(std::vector<SmLaunch> *v) { g_captureLaunches = v; }
        ~CaptureScope() { g_captureLaunches = nullptr; }
    } captureScope(fastOk ? &captured : nullptr);
    RegisterBuiltinExecutors();
    if (c->env.entryLogEnable)
        HCCL_RUN_INFO("Entry-%s: tag[%s] in[%p] out[%p] count[%llu] dtype[%s] op[%s] root[%u] peer[%u] stream[%p] rank[%u/%u]", CmdName(p.opType),
                      p.tag.c_str(), p.inputPtr, p.outputPtr, (unsigned long long)p.count, DataTypeName(p.dtype), ReduceOpName(p.reduceOp), p.root,
                      p.peer, (void *)p.stream, c->rank, c->nranks);
    if (c->nranks == 1) {
        CHK_RET(SingleRankProc(c, p));
        c->counters.ops++;
        return HCCL_SUCCESS;
    }
    std::vector<HcclCommEngine> excluded;
    std::string stickyKey = p.tag + "|" + std::to_string((int)p.dtype) + "|" + std::to_string((int)p.reduceOp);
    {
        std::lock_guard<std::mutex> lk(c->ctxMu);
        auto it = c->stickyFallback.find(stickyKey);
        if (it != c->stickyFallback.end()) {
            // everything tried before the engine that finally worked stays excluded
            for (HcclCommEngine e : {HCCL_ENGINE_NVLS, HCCL_ENGINE_SM, HCCL_ENGINE_COPY_ENGINE}) {
                if ((int)e == it->second) break;
                excluded.push_back(e);
            }
        }
    }
    HcclResult res = HCCL_E_INTERNAL;
    const uint64_t devSeqBefore = c->devOpIssued.load();
    bool resourceFallback = false;   // only a missing resource is remembered; a call-specific "not supported" is not
    for (int attempt = 0; attempt < 4; ++attempt) {
        CHK_RET(SelectAlgorithm(c, p, excluded));
        CHK_RET(CheckOpConsistency(c, p));
        std::unique_ptr<ExecutorBase> exec = ExecutorRegistry::Instance().Create(p.opType, p.algName);
        if (!exec) {
            HCCL_ERROR("algorithm %s is not registered for %s", p.algName.c_str(), CmdName(p.opType));
            return HCCL_E_NOT_FOUND;
        }
        NvtxPush(p.algTag.c_str());
        res = dropThisOp ? HCCL_SUCCESS : exec->Orchestrate(c, p);
        NvtxPop();
        if (res != HCCL_E_UNAVAIL && res != HCCL_E_NOT_SUPPORT) break;
        if (p.engine == HCCL_ENGINE_HOST || p.engine == HCCL_ENGINE_COPY_ENGINE) break;   // nothing below to fall back to
        if (res == HCCL_E_NOT_SUPPORT) HCCL_INFO("%s on engine %s does not take this call; falling back", p.algName.c_str(), EngineName(p.engine));
        else HCCL_WARNING("%s on engine %s is unavailable (%d); falling back", p.algName.c_str(), EngineName(p.engine), (int)res);
        if (res == HCCL_E_UNAVAIL) resourceFallback = true;
        excluded.push_back(p.engine);
        c->counters.fallbacks++;
    }
    if (res == HCCL_SUCCESS && resourceFallback) {
        std::lock_guard<std::mutex> lk(c->ctxMu);
        c->stickyFallback[stickyKey] = (int)p.engine;
    }
    OpRecord rec{};
    rec.seq = c->counters.ops++;
    rec.opType = p.opType;
    rec.dtype = p.dtype;
    rec.reduceOp = p.reduceOp;
    rec.count = p.count;
    rec.root = p.root;
    rec.engine = (uint32_t)p.engine;
    snprintf(rec.algName, sizeof(rec.algName), "%s", p.algName.c_str());
    rec.beginNs = begin;
    rec.endNs = NowNs();
    rec.devSeq = (uint32_t)devSeqBefore; rec.devLaunches = (uint32_t)(c->devOpIssued.load() - devSeqBefore);
    RecordOp(c, rec);
    c->counters.bytes += p.DataBytes();
    uint64_t *histSlot;
    {
        std::lock_guard<std::mutex> lk(c->counters.mu);
        histSlot = &c->counters.algoHistogram[p.algName];
        ++*histSlot;
    }
    if (fastOk && res == HCCL_SUCCESS && !dropThisOp && !captured.empty() && (p.engine == HCCL_ENGINE_SM || p.engine == HCCL_ENGINE_NVLS)) {
        if (!c->fastOps) c->fastOps = std::make_shared<FastCache>();
        auto *fc = static_cast<FastCache *>(c->fastOps.get());
        if (fc->map.size() >= kFastCacheCap) {
            // drop the least recently used fifth, as the reference's launch cache does
            std::vector<uint64_t> uses;
            uses.reserve(fc->map.size());
            for (auto &kv : fc->map) uses.push_back(kv.second.lastUse);
            std::nth_element(uses.begin(), uses.begin() + uses.size() / 5, uses.end());
            const uint64_t cut = uses[uses.size() / 5];
            for (auto it = fc->map.begin(); it != fc->map.end();) it = it->second.lastUse <= cut ? fc->map.erase(it) : std::next(it);
        }
        fc->map[fkey] = FastEntry{p.algName, p.engine, std::move(captured), g_selectGeneration.load(), histSlot, ++fc->tick};
    }
    if (c->env.entryLogEnable)
        HCCL_RUN_INFO("Exit-%s: alg[%s] engine[%s] ret[%d] host_us[%llu]", CmdName(p.opType), p.algName.c_str(), EngineName(p.engine), (int)res,
                      (unsigned long long)((rec.endNs - rec.beginNs) / 1000));
    return res;
}

}  // namespace hccl
