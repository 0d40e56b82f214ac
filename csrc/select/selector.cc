#include "selector.h"
#include "../exec/op_common.h"
#include "../exec/slice_planner.h"
#include <dlfcn.h>
#include <algorithm>
#include <mutex>
#include <fstream>
#include <sstream>
#include <tuple>
#include "../common/dtype.h"
#include "../common/log.h"

namespace hccl {

// ------------------------------------------------------------------------------------------------ registry
SelectorRegistry &SelectorRegistry::Instance()
{
    static SelectorRegistry r;
    return r;
}
void SelectorRegistry::Register(HcclCMDType op, int priority, std::function<AutoSelectorBase *()> factory)
{
    auto &v = map_[op];
    v.push_back({priority, std::move(factory), nullptr});
    std::stable_sort(v.begin(), v.end(), [](const Entry &a, const Entry &b) { return a.priority < b.priority; });
}
std::vector<AutoSelectorBase *> SelectorRegistry::Get(HcclCMDType op)
{
    static std::mutex mu;                    // selectors are instantiated on first use; ranks of one process race here
    std::lock_guard<std::mutex> lk(mu);
    std::vector<AutoSelectorBase *> out;
    auto it = map_.find(op);
    if (it == map_.end()) return out;
    for (auto &e : it->second) {
        if (!e.inst) e.inst = e.factory();
        out.push_back(e.inst);
    }
    return out;
}

bool NvlsSupports(HcclDataType t, HcclReduceOp op)
{
    if (t == HCCL_DATA_TYPE_FP32) return op == HCCL_REDUCE_SUM;
    if (t == HCCL_DATA_TYPE_FP16 || t == HCCL_DATA_TYPE_BFP16) return op == HCCL_REDUCE_SUM || op == HCCL_REDUCE_MAX || op == HCCL_REDUCE_MIN;
    return false;
}

bool SmReduceSupports(HcclDataType t, HcclReduceOp op)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_INT64:
        case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_FP32: case HCCL_DATA_TYPE_FP64:
        case HCCL_DATA_TYPE_BFP16: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_UINT32: return op <= HCCL_REDUCE_MIN;
        default: return false;
    }
}

// ------------------------------------------------------------------------------------------------ tuning table
TuningTable &TuningTable::Instance()
{
    static TuningTable t;
    return t;
}
TuningTable::TuningTable() { ResetToBuiltin(); }

void TuningTable::Set(HcclCMDType op, uint32_t nranks, HcclCommEngine engine, std::vector<TuningRow> rows)
{
    std::sort(rows.begin(), rows.end(), [](const TuningRow &a, const TuningRow &b) { return a.maxBytes < b.maxBytes; });
    rows_[Key{op, nranks, engine}] = std::move(rows);
    BumpSelectionGeneration();
}

const TuningRow *TuningTable::Lookup(HcclCMDType op, uint32_t nranks, HcclCommEngine engine, uint64_t bytes) const
{
    auto it = rows_.find(Key{op, nranks, engine});
    if (it == rows_.end()) it = rows_.find(Key{op, 0, engine});
    if (it == rows_.end()) return nullptr;
    for (const TuningRow &r : it->second) if (bytes <= r.maxBytes) return &r;
    return it->second.empty() ? nullptr : &it->second.back();
}

// Built-in priors. Sizes are the payload the selector sees (OpParam::DataBytes). They start from HCCL's
// crossovers (one-shot below 128 KB..8 MB depending on engine, "small" below 512 KB) and are replaced by the
// measured table when HCCL_TUNING_FILE is set.
void TuningTable::ResetToBuiltin()
{
    rows_.clear();
    const uint64_t INF = ~0ull;
    Set(HCCL_CMD_ALLREDUCE, 0, HCCL_ENGINE_SM, {{256u << 10, "SmAllReduceMesh1DOneShot", 0}, {INF, "SmAllReduceMesh1DTwoShot", 0}});
    Set(HCCL_CMD_ALLREDUCE, 0, HCCL_ENGINE_NVLS, {{512u << 10, "NvlsAllReduceOneShot", 0}, {128u << 20, "NvlsAllReduceTwoShot", 0}, {INF, "NvlsAllReducePipelined", 0}});
    Set(HCCL_CMD_ALLGATHER, 0, HCCL_ENGINE_SM, {{INF, "SmAllGatherMesh1D", 0}});
    Set(HCCL_CMD_REDUCE_SCATTER, 0, HCCL_ENGINE_SM, {{INF, "SmReduceScatterMesh1D", 0}});
    Set(HCCL_CMD_REDUCE_SCATTER, 0, HCCL_ENGINE_NVLS, {{32u << 20, "NvlsReduceScatter", 0}, {INF, "NvlsReduceScatterPipelined", 0}});
    Set(HCCL_CMD_BROADCAST, 0, HCCL_ENGINE_SM, {{INF, "SmBroadcastMesh1D", 0}});
    Set(HCCL_CMD_BROADCAST, 0, HCCL_ENGINE_NVLS, {{INF, "NvlsBroadcast", 0}});
    Set(HCCL_CMD_REDUCE, 0, HCCL_ENGINE_SM, {{INF, "SmReduceMesh1D", 0}});
    Set(HCCL_CMD_SCATTER, 0, HCCL_ENGINE_SM, {{INF, "SmScatterMesh1D", 0}});
    Set(HCCL_CMD_ALLTOALL, 0, HCCL_ENGINE_SM, {{INF, "SmAlltoAllMesh1D", 0}});
    Set(HCCL_CMD_ALLTOALLV, 0, HCCL_ENGINE_SM, {{INF, "SmAlltoAllVMesh1D", 0}});
    Set(HCCL_CMD_ALLTOALLVC, 0, HCCL_ENGINE_SM, {{INF, "SmAlltoAllVCMesh1D", 0}});
    Set(HCCL_CMD_ALLGATHER_V, 0, HCCL_ENGINE_SM, {{INF, "SmAllGatherVMesh1D", 0}});
    Set(HCCL_CMD_REDUCE_SCATTER_V, 0, HCCL_ENGINE_SM, {{INF, "SmReduceScatterVMesh1D", 0}});
    Set(HCCL_CMD_BARRIER, 0, HCCL_ENGINE_SM, {{INF, "SmBarrierMesh1D", 0}});
    Set(HCCL_CMD_SEND, 0, HCCL_ENGINE_SM, {{INF, "SmSend", 0}});
    Set(HCCL_CMD_RECEIVE, 0, HCCL_ENGINE_SM, {{INF, "SmRecv", 0}});
    Set(HCCL_CMD_BATCH_SEND_RECV, 0, HCCL_ENGINE_SM, {{INF, "SmBatchSendRecv", 0}});
}

HcclResult TuningTable::LoadText(const std::string &text)
{
    std::map<Key, std::vector<TuningRow>> fresh;
    std::istringstream is(text);
    std::string line;
    int lineNo = 0;
    while (std::getline(is, line)) {
        ++lineNo;
        size_t h = line.find('#');
        if (h != std::string::npos) line = line.substr(0, h);
        std::istringstream ls(line);
        std::string opName, engName, maxStr, alg;
        uint32_t n, ctas;
        if (!(ls >> opName)) continue;
        if (!(ls >> n >> engName >> maxStr >> alg >> ctas)) { HCCL_ERROR("tuning table line %d: expected 6 fields", lineNo); return HCCL_E_PARA; }
        HcclCMDType op;
        HcclCommEngine eng;
        if (!ParseOpName(opName, &op) || !ParseEngineName(engName, &eng)) { HCCL_ERROR("tuning table line %d: unknown op/engine", lineNo); return HCCL_E_PARA; }
        uint64_t maxBytes = maxStr == "inf" ? ~0ull : strtoull(maxStr.c_str(), nullptr, 10);
        fresh[Key{op, n, eng}].push_back({maxBytes, alg, ctas});
    }
    for (auto &kv : fresh) Set(kv.first.op, kv.first.n, kv.first.e, kv.second);
    return HCCL_SUCCESS;
}

HcclResult TuningTable::LoadFile(const std::string &path)
{
    std::ifstream f(path);
    if (!f) { HCCL_ERROR("tuning table %s cannot be opened", path.c_str()); return HCCL_E_OPEN_FILE_FAILURE; }
    std::stringstream ss;
    ss << f.rdbuf();
    return LoadText(ss.str());
}

HcclResult TuningTable::LoadConfigured(const std::string &envFile)
{
    static std::once_flag once;
    static HcclResult result = HCCL_SUCCESS;
    std::call_once(once, [&] {
        Dl_info info;
        if (dladdr((const void *)&TuningTable::Instance, &info) && info.dli_fname) {
            std::string lib = info.dli_fname;
            size_t slash = lib.rfind('/');
            std::string packaged = (slash == std::string::npos ? std::string(".") : lib.substr(0, slash)) + "/../tuning/b200.txt";
            std::ifstream f(packaged);
            if (f) {
                std::stringstream ss;
                ss << f.rdbuf();
                if (LoadText(ss.str()) == HCCL_SUCCESS) HCCL_RUN_INFO("tuning table: loaded %s", packaged.c_str());
                else HCCL_WARNING("tuning table: %s is malformed and was ignored", packaged.c_str());
            }
        }
        if (!envFile.empty()) result = LoadFile(envFile);
    });
    return result;
}

std::string TuningTable::Dump() const
{
    std::ostringstream os;
    for (auto &kv : rows_)
        for (auto &r : kv.second) {
            os << CmdName(kv.first.op) << " " << kv.first.n << " " << EngineName(kv.first.e) << " ";
            if (r.maxBytes == ~0ull) os << "inf"; else os << r.maxBytes;
            os << " " << r.algName << " " << r.ctas << "\n";
        }
    return os.str();
}

// ------------------------------------------------------------------------------------------------ IR algorithm choice
// Used by the HOST and COPY_ENGINE engines. `forced` comes from HCCL_ALGO level1 (ring / NHR / fullmesh ...).
const char *IrAlgoFor(HcclCMDType op, AlgoType forced, uint64_t bytes, uint32_t nranks, uint64_t cclBytes)
{
    bool ring = forced == AlgoType::RING;
    bool nhr = forced == AlgoType::NHR || forced == AlgoType::NHR_V1 || forced == AlgoType::NB || forced == AlgoType::HDR;
    switch (op) {
        case HCCL_CMD_ALLREDUCE:
            if (ring) return "InsAllReduceRing";
            if (nhr) return "InsAllReduceNHR";
            // one-shot while the whole payload fits N times into scratch and is small (reference prior: 8 MB on the host engine)
            if (bytes <= (8u << 20) && bytes * nranks + (64u << 10) <= cclBytes && bytes <= (256u << 10)) return "InsAllReduceMesh1DOneShot";
            return "InsAllReduceMesh1DTwoShot";
        case HCCL_CMD_ALLGATHER: return ring ? "InsAllGatherRing" : nhr ? "InsAllGatherNHR" : "InsAllGatherMesh1D";
        case HCCL_CMD_REDUCE_SCATTER: return ring ? "InsReduceScatterRing" : nhr ? "InsReduceScatterNHR" : "InsReduceScatterMesh1D";
        case HCCL_CMD_BROADCAST: return nhr ? "InsBroadcastNHR" : bytes <= (64u << 10) ? "InsBroadcastMesh1DOneShot" : "InsBroadcastMesh1DTwoShot";
        case HCCL_CMD_REDUCE: return nhr ? "ReduceNHR" : bytes <= (512u << 10) ? "ReduceMesh1D" : "ReduceMesh1DTwoShot";
        case HCCL_CMD_SCATTER: return nhr ? "InsScatterNHR" : "InsScatterMesh1D";
        case HCCL_CMD_ALLTOALL: return "InsAlltoAllMesh1D";
        case HCCL_CMD_ALLTOALLV: return "InsAlltoAllVMesh1D";
        case HCCL_CMD_ALLTOALLVC: return "InsAlltoAllVCMesh1D";
        case HCCL_CMD_ALLGATHER_V: return "InsAllGatherVMesh1D";
        case HCCL_CMD_REDUCE_SCATTER_V: return "InsReduceScatterVMesh1D";
        case HCCL_CMD_BARRIER: return nhr ? "InsBarrierNHR" : "InsBarrierMesh1D";
        case HCCL_CMD_SEND: return "InsSend";
        case HCCL_CMD_RECEIVE: return "InsRecv";
        case HCCL_CMD_BATCH_SEND_RECV: return "InsBatchSendRecv";
        default: return nullptr;
    }
}

// ------------------------------------------------------------------------------------------------ cascade
static bool Excluded(const SelectorCtx &ctx, HcclCommEngine e)
{
    return std::find(ctx.excluded.begin(), ctx.excluded.end(), e) != ctx.excluded.end();
}

namespace {
bool NvlsSupportsZc(HcclDataType dt, HcclReduceOp op)
{
    if (dt == HCCL_DATA_TYPE_FP32) return op == HCCL_REDUCE_SUM;
    if (dt == HCCL_DATA_TYPE_BFP16 || dt == HCCL_DATA_TYPE_FP16) return op == HCCL_REDUCE_SUM || op == HCCL_REDUCE_MAX || op == HCCL_REDUCE_MIN;
    return false;
}
bool ZeroCopyApplies(const SelectorCtx &ctx, OpParam &p)
{
    static const bool enabled = [] { const char *e = getenv("HCCL_ZERO_COPY"); return e ? atoi(e) != 0 : true; }();
    static const uint64_t minBytes = [] { const char *e = getenv("HCCL_ZERO_COPY_MIN_BYTES"); return e ? (uint64_t)strtoull(e, nullptr, 0) : (1ull << 20); }();
    if (!enabled || p.mode != OpMode::OPBASE) return false;
    const uint32_t n = ctx.topo->nranks;
    const uint64_t bytes = p.count * DataTypeSize(p.dtype);
    if (bytes < minBytes || bytes % 16 || ((uintptr_t)p.inputPtr & 15u) || ((uintptr_t)p.outputPtr & 15u)) return false;
    const char *base = nullptr;
    bool reduces = false;
    switch (p.opType) {
        case HCCL_CMD_ALLREDUCE:
            if (!CommRegisteredOffset(ctx.comm, p.inputPtr, bytes, nullptr) || !CommRegisteredOffset(ctx.comm, p.outputPtr, bytes, nullptr)) return false;
            base = "AllReduce"; reduces = true; break;
        case HCCL_CMD_REDUCE_SCATTER:
            if (!CommRegisteredOffset(ctx.comm, p.inputPtr, bytes * n, nullptr)) return false;
            base = "ReduceScatter"; reduces = true; break;
        case HCCL_CMD_ALLGATHER:
            if (!CommRegisteredOffset(ctx.comm, p.outputPtr, bytes * n, nullptr)) return false;
            base = "AllGather"; break;
        case HCCL_CMD_BROADCAST:
            if (!CommRegisteredOffset(ctx.comm, p.outputPtr, bytes, nullptr)) return false;
            base = "Broadcast"; break;
        default: return false;
    }
    HcclCommEngine want = ctx.env->expansionMode;
    auto perOp = ctx.env->expansionModePerOp.find(p.opType);
    if (perOp != ctx.env->expansionModePerOp.end()) want = perOp->second;
    if (want == HCCL_ENGINE_COPY_ENGINE || want == HCCL_ENGINE_HOST) return false;
    bool nv = ctx.nvls && want != HCCL_ENGINE_SM && (!reduces || (ctx.env->deterministic == Deterministic::OFF && NvlsSupportsZc(p.dtype, p.reduceOp)));
    if (reduces && !nv) {
        // the peer-load form reduces in rank order with fp32 accumulation: every reducible type of the SM engine
        switch (p.dtype) {
            case HCCL_DATA_TYPE_FP32: case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_INT64:
            case HCCL_DATA_TYPE_FP64: case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_INT16: break;
            default: return false;
        }
    }
    p.engine = nv ? HCCL_ENGINE_NVLS : HCCL_ENGINE_SM;
    p.algName = std::string(nv ? "Nvls" : "Sm") + base + "ZeroCopy";
    return true;
}
}  // namespace

SelectorStatus AutoSelectorBase::Select(const SelectorCtx &ctx, OpParam &param) const
{
    // explicit algorithm name wins (engine inferred from the prefix)
    auto nameIt = ctx.env->algoNamePerOp.find(param.opType);
    if (nameIt != ctx.env->algoNamePerOp.end() && ctx.excluded.empty()) {
        const std::string &nm = nameIt->second;
        param.algName = nm;
        if (nm.rfind("Nvls", 0) == 0) param.engine = HCCL_ENGINE_NVLS;
        else if (nm.rfind("Sm", 0) == 0) param.engine = HCCL_ENGINE_SM;
        else param.engine = ctx.cuda ? HCCL_ENGINE_COPY_ENGINE : HCCL_ENGINE_HOST;
        return SelectorStatus::MATCH;
    }
    // Registered windows on the rank-crossing side of the transfer: no staging through the scratch buffer at all. Chosen from
    // HCCL_ZERO_COPY_MIN_BYTES up (default 1 MB; below that the staged one-shot kernels have one synchronisation less);
    // HCCL_ZERO_COPY=0 switches the rule off. Every rank decides from its own pointers: buffers that come from the same
    // symmetric allocation give the same answer everywhere, and the consistency exchange compares the algorithm names.
    if (ctx.cuda && ctx.comm && ctx.excluded.empty() && ZeroCopyApplies(ctx, param)) return SelectorStatus::MATCH;
    HcclCommEngine want = ctx.env->expansionMode;
    auto perOp = ctx.env->expansionModePerOp.find(param.opType);
    if (perOp != ctx.env->expansionModePerOp.end()) want = perOp->second;
    if (!ctx.cuda) {
        param.engine = HCCL_ENGINE_HOST;
        return SelectIr(ctx, param);
    }
    std::vector<HcclCommEngine> order;
    if (want != HCCL_ENGINE_DEFAULT && want != HCCL_ENGINE_HOST) order.push_back(want);
    for (HcclCommEngine e : {HCCL_ENGINE_NVLS, HCCL_ENGINE_SM, HCCL_ENGINE_COPY_ENGINE})
        if (std::find(order.begin(), order.end(), e) == order.end()) {
            // an explicit SM / COPY_ENGINE request must not be upgraded to NVLS
            if (e == HCCL_ENGINE_NVLS && want != HCCL_ENGINE_DEFAULT && want != HCCL_ENGINE_NVLS) continue;
            order.push_back(e);
        }
    for (HcclCommEngine e : order) {
        if (Excluded(ctx, e)) continue;
        SelectorStatus st = SelectorStatus::NOT_MATCH;
        param.engine = e;
        if (e == HCCL_ENGINE_NVLS) {
            if (!ctx.nvls || ctx.env->deterministic != Deterministic::OFF) continue;   // switch reduction order is not ours to fix
            st = SelectNvls(ctx, param);
        } else if (e == HCCL_ENGINE_SM) st = SelectSm(ctx, param);
        else {
            // Point-to-point schedules use several queues whose waits resolve through the peer; as stream work on one GPU
            // those would be separate launches that depend on one another, which nothing guarantees to co-run. The SM
            // engine serves them in a single launch instead.
            if (param.opType == HCCL_CMD_SEND || param.opType == HCCL_CMD_RECEIVE || param.opType == HCCL_CMD_BATCH_SEND_RECV) continue;
            st = SelectIr(ctx, param);
        }
        if (st == SelectorStatus::MATCH) return st;
    }
    return SelectorStatus::NOT_MATCH;
}

HcclResult ExecuteSelector(const SelectorCtx &ctx, OpParam &param)
{
    auto sels = SelectorRegistry::Instance().Get(param.opType);
    if (sels.empty()) { HCCL_ERROR("no selector registered for %s", CmdName(param.opType)); return HCCL_E_NOT_FOUND; }
    for (AutoSelectorBase *s : sels) {
        if (s->Select(ctx, param) == SelectorStatus::MATCH) {
            HCCL_MOD_DEBUG(MOD_ALG, "selected %s on %s for %s bytes=%llu", param.algName.c_str(), EngineName(param.engine),
                           CmdName(param.opType), (unsigned long long)param.DataBytes());
            return HCCL_SUCCESS;
        }
    }
    HCCL_ERROR("no algorithm matches %s dtype=%s op=%s bytes=%llu", CmdName(param.opType), DataTypeName(param.dtype),
               ReduceOpName(param.reduceOp), (unsigned long long)param.DataBytes());
    return HCCL_E_NOT_SUPPORT;
}

// ------------------------------------------------------------------------------------------------ per-op selectors
namespace {

AlgoType ForcedAlgo(const SelectorCtx &ctx, HcclCMDType op)
{
    auto it = ctx.env->algoPerOp.find(op);
    const AlgoLevels &lv = it != ctx.env->algoPerOp.end() ? it->second : ctx.env->algo;
    // one NVSwitch level: level1 names the flat algorithm a user asks for; level0 is "NA" by definition
    return lv.level[1] != AlgoType::DEFAULT ? lv.level[1] : lv.level[0] == AlgoType::NA ? AlgoType::DEFAULT : lv.level[0];
}

SelectorStatus FromTable(const SelectorCtx &ctx, OpParam &p, HcclCommEngine eng)
{
    const TuningRow *row = TuningTable::Instance().Lookup(p.opType, ctx.topo->nranks, eng, p.DataBytes());
    if (!row || row->algName == "none") return SelectorStatus::NOT_MATCH;   // "none": this engine passes on the size range
    p.algName = row->algName;
    return SelectorStatus::MATCH;
}

SelectorStatus IrDefault(const SelectorCtx &ctx, OpParam &p)
{
    AlgoType forced = ForcedAlgo(ctx, p.opType);
    // HCCL_DETERMINISTIC=strict (the reference's order-preserved executors, reference:
    // src/ops/all_reduce/selector/all_reduce_auto_selector.cc:360-371): reductions use the flat mesh templates, whose
    // fixed rank order makes an element's bits independent of count, chunking, topology level split and of which of the
    // one-shot / two-shot forms the size selects. Ring / NHR / sequence requests are overridden for reductions.
    const bool reduces = p.opType == HCCL_CMD_ALLREDUCE || p.opType == HCCL_CMD_REDUCE_SCATTER || p.opType == HCCL_CMD_REDUCE_SCATTER_V ||
                         p.opType == HCCL_CMD_REDUCE;
    const bool strict = ctx.env->deterministic == Deterministic::STRICT && reduces;
    if (strict) forced = AlgoType::FULLMESH;
    // HCCL_BIRS_ENABLE=1 (the reference's experimental batch-invariant ReduceScatter for its 2-D topology, reference:
    // experimental/ops/reduce_scatter/birs, docs/en/rfcs/0001-add-batch-invariant-reducescatter.md): an element's bits must not
    // depend on how many elements travel with it. On two levels that is the sequence executor (every element is summed inside the
    // server in rank order, then across the servers in server order); the parallel executor is excluded because its cut between
    // the level orders moves with the count. On one level it is the rank-ordered mesh.
    const char *birsEnv = getenv("HCCL_BIRS_ENABLE");
    const bool birs = birsEnv && birsEnv[0] == '1';
    const bool batchInvariant = birs && p.opType == HCCL_CMD_REDUCE_SCATTER;
    if (batchInvariant && ctx.topo->numLevels == 1) forced = AlgoType::FULLMESH;
    // multi-level topologies use the sequence executors for the ops that have one
    if (ctx.topo->numLevels >= 2 && forced == AlgoType::DEFAULT && !ctx.cuda && !strict && !batchInvariant &&
        (p.opType == HCCL_CMD_ALLREDUCE || p.opType == HCCL_CMD_ALLGATHER || p.opType == HCCL_CMD_REDUCE_SCATTER)) {
        // Two levels and an engine that runs several queues: when the slice planner prices the form that keeps both levels
        // busy at least a tenth below the sequential one, use it (HCCL_PARALLEL_EXECUTOR=0 keeps the sequence executors).
        static const bool allow = [] { const char *e = getenv("HCCL_PARALLEL_EXECUTOR"); return !(e && e[0] == '0'); }();
        AlgHierarchyInfo h;
        if (allow && TopoMatch(*ctx.topo, TopoMatchKind::TWO_LEVEL, &h) == HCCL_SUCCESS && h.levelRanks.size() == 2 && ctx.topo->levelBandwidth.size() >= 2) {
            SlicePlan sp;
            const PipeOp po = p.opType == HCCL_CMD_ALLREDUCE ? PipeOp::ALLREDUCE : p.opType == HCCL_CMD_ALLGATHER ? PipeOp::ALLGATHER : PipeOp::REDUCE_SCATTER;
            if (PlanSlices(po, AxisSpec{(uint32_t)h.levelRanks[0].size(), ctx.topo->levelBandwidth[0], 2.0},
                           AxisSpec{(uint32_t)h.levelRanks[1].size(), FoldedUpperBandwidth(*ctx.topo, 50.0), 5.0}, p.DataBytes(), 512, 4, &sp) == HCCL_SUCCESS &&
                (sp.shares.size() == 2 || sp.shares[0].steps > 1) && sp.parallelUs < 0.9 * sp.sequenceUs) {
                p.algName = po == PipeOp::ALLREDUCE ? "InsAllReduceParallelMesh1DMesh1D" : po == PipeOp::ALLGATHER ? "InsAllGatherParallelMesh1DMesh1D" : "InsReduceScatterParallelMesh1DMesh1D";
                return SelectorStatus::MATCH;
            }
        }
    }
    if (ctx.topo->numLevels > 1 && forced == AlgoType::DEFAULT) {
        if (p.opType == HCCL_CMD_ALLREDUCE) { p.algName = "InsAllReduceSequenceMesh1DNhr"; return SelectorStatus::MATCH; }
        if (p.opType == HCCL_CMD_ALLGATHER) { p.algName = "InsAllGatherSequenceNhrMesh1D"; return SelectorStatus::MATCH; }
        if (p.opType == HCCL_CMD_REDUCE_SCATTER) { p.algName = "InsReduceScatterSequenceMesh1DNhr"; return SelectorStatus::MATCH; }
        // rooted operators: the data crosses the servers once, through the root's column
        if (ctx.topo->symmetric) {
            if (p.opType == HCCL_CMD_BROADCAST) { p.algName = "InsBroadcastSequenceMesh1DMesh1D"; return SelectorStatus::MATCH; }
            if (p.opType == HCCL_CMD_REDUCE) { p.algName = "InsReduceSequenceMesh1DMesh1D"; return SelectorStatus::MATCH; }
            if (p.opType == HCCL_CMD_SCATTER) { p.algName = "InsScatterSequenceMesh1DMesh1D"; return SelectorStatus::MATCH; }
            if (p.opType == HCCL_CMD_BARRIER) { p.algName = "InsBarrierSequenceMesh1DMesh1D"; return SelectorStatus::MATCH; }
        }
    }
    const char *nm = IrAlgoFor(p.opType, forced, p.DataBytes(), ctx.topo->nranks, ctx.cclBytes);
    if (!nm) return SelectorStatus::NOT_MATCH;
    p.algName = nm;
    return SelectorStatus::MATCH;
}

class ReduceFamilySelector : public AutoSelectorBase {   // AllReduce, ReduceScatter(V), Reduce
protected:
    SelectorStatus SelectNvls(const SelectorCtx &ctx, OpParam &p) const override
    {
        if (!NvlsSupports(p.dtype, p.reduceOp)) return SelectorStatus::NOT_MATCH;
        if (ForcedAlgo(ctx, p.opType) == AlgoType::RING) return SelectorStatus::NOT_MATCH;
        return FromTable(ctx, p, HCCL_ENGINE_NVLS);
    }
    SelectorStatus SelectSm(const SelectorCtx &ctx, OpParam &p) const override
    {
        if (!SmReduceSupports(p.dtype, p.reduceOp)) return SelectorStatus::NOT_MATCH;
        AlgoType f = ForcedAlgo(ctx, p.opType);
        if (f == AlgoType::RING && p.opType == HCCL_CMD_ALLREDUCE) { p.algName = "SmAllReduceRing"; return SelectorStatus::MATCH; }
        if (f == AlgoType::RING || f == AlgoType::NHR) return SelectorStatus::NOT_MATCH;   // those live in the IR engines
        return FromTable(ctx, p, HCCL_ENGINE_SM);
    }
    SelectorStatus SelectIr(const SelectorCtx &ctx, OpParam &p) const override { return IrDefault(ctx, p); }
};

class CopyFamilySelector : public AutoSelectorBase {     // everything that only moves bytes
protected:
    SelectorStatus SelectNvls(const SelectorCtx &ctx, OpParam &p) const override
    {
        if (p.opType == HCCL_CMD_ALLGATHER || p.opType == HCCL_CMD_ALLGATHER_V) return FromTable(ctx, p, HCCL_ENGINE_NVLS);
        if (p.opType != HCCL_CMD_BROADCAST) return SelectorStatus::NOT_MATCH;
        if (IsSmallData(p.DataBytes())) return SelectorStatus::NOT_MATCH;   // pull from root wins on latency
        return FromTable(ctx, p, HCCL_ENGINE_NVLS);
    }
    SelectorStatus SelectSm(const SelectorCtx &ctx, OpParam &p) const override
    {
        AlgoType f = ForcedAlgo(ctx, p.opType);
        if (f == AlgoType::RING || f == AlgoType::NHR) return SelectorStatus::NOT_MATCH;
        return FromTable(ctx, p, HCCL_ENGINE_SM);
    }
    SelectorStatus SelectIr(const SelectorCtx &ctx, OpParam &p) const override { return IrDefault(ctx, p); }
};

// MC2 / MoE ops always run as one fused SM kernel; the selector only names it.
class FusedSelector : public AutoSelectorBase {
protected:
    SelectorStatus SelectSm(const SelectorCtx &, OpParam &p) const override
    {
        switch (p.opType) {
            case HCCL_CMD_ALLGATHER_MATMUL: p.algName = "SmAllGatherMatmulFused"; break;
            case HCCL_CMD_MATMUL_REDUCE_SCATTER: p.algName = "SmMatmulReduceScatterFused"; break;
            case HCCL_CMD_MATMUL_ALLREDUCE: p.algName = "SmMatmulAllReduceFused"; break;
            case HCCL_CMD_MOE_DISPATCH: p.algName = "SmMoeDispatchFused"; break;
            case HCCL_CMD_MOE_COMBINE: p.algName = "SmMoeCombineFused"; break;
            default: return SelectorStatus::NOT_MATCH;
        }
        return SelectorStatus::MATCH;
    }
};

REGISTER_SELECTOR_BY_OPTYPE(HCCL_CMD_ALLREDUCE, 10, ReduceFamilySelector);
class ReduceScatterSelector : public ReduceFamilySelector {};
class ReduceScatterVSelector : public ReduceFamilySelector {};
class ReduceSelector : public ReduceFamilySelector {};
REGISTER_SELECTOR_BY_OPTYPE(HCCL_CMD_REDUCE_SCATTER, 10, ReduceScatterSelector);
REGISTER_SELECTOR_BY_OPTYPE(HCCL_CMD_REDUCE_SCATTER_V, 10, ReduceScatterVSelector);
REGISTER_SELECTOR_BY_OPTYPE(HCCL_CMD_REDUCE, 10, ReduceSelector);
#define COPY_SEL(cls, op) class cls : public CopyFamilySelector {}; REGISTER_SELECTOR_BY_OPTYPE(op, 10, cls)
COPY_SEL(AllGatherSelector, HCCL_CMD_ALLGATHER);
COPY_SEL(AllGatherVSelector, HCCL_CMD_ALLGATHER_V);
COPY_SEL(BroadcastSelector, HCCL_CMD_BROADCAST);
COPY_SEL(ScatterSelector, HCCL_CMD_SCATTER);
COPY_SEL(AlltoAllSelector, HCCL_CMD_ALLTOALL);
COPY_SEL(AlltoAllVSelector, HCCL_CMD_ALLTOALLV);
COPY_SEL(AlltoAllVCSelector, HCCL_CMD_ALLTOALLVC);
COPY_SEL(SendSelector, HCCL_CMD_SEND);
COPY_SEL(RecvSelector, HCCL_CMD_RECEIVE);
COPY_SEL(BatchSendRecvSelector, HCCL_CMD_BATCH_SEND_RECV);
COPY_SEL(BarrierSelector, HCCL_CMD_BARRIER);
#define FUSED_SEL(cls, op) class cls : public FusedSelector {}; REGISTER_SELECTOR_BY_OPTYPE(op, 18, cls)
FUSED_SEL(AgMatmulSelector, HCCL_CMD_ALLGATHER_MATMUL);
FUSED_SEL(MatmulRsSelector, HCCL_CMD_MATMUL_REDUCE_SCATTER);
FUSED_SEL(MatmulArSelector, HCCL_CMD_MATMUL_ALLREDUCE);
FUSED_SEL(MoeDispatchSelector, HCCL_CMD_MOE_DISPATCH);
FUSED_SEL(MoeCombineSelector, HCCL_CMD_MOE_COMBINE);

}  // namespace

// Referenced from the dispatch core so that a static-library link keeps this translation unit (and with it the
// registrations above).
void EnsureSelectorsLinked() {}

}  // namespace hccl
