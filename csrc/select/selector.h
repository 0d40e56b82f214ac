// Algorithm selection: engine cascade + per-op auto selectors + a tuning table of measured crossovers.
//
// Structure follows HCCL's (reference: src/ops/op_common/selector/auto_selector_base.cc:17-68 engine cascade
// CCU_MS -> CCU_SCHED -> AIV -> AICPU; selector_registry.h:52 REGISTER_SELECTOR_BY_OPTYPE with priorities;
// execute_selector.cc:21-55 walks the registry; per-op thresholds such as
// src/ops/all_reduce/selector/all_reduce_auto_selector.cc:18-35,578-597). The cascade here is
// NVLS -> SM -> COPY_ENGINE on CUDA communicators and HOST on simulated ones; the size thresholds come from a
// table keyed by (op, ranks, dtype width) that a sweep on the target box regenerates (HCCL_TUNING_FILE).
#pragma once
#include <functional>
#include <map>
#include <string>
#include <vector>
#include "../core/comm.h"
#include "../exec/op_param.h"

namespace hccl {

enum class SelectorStatus : uint8_t { MATCH = 0, NOT_MATCH = 1 };

struct SelectorCtx {
    Comm *comm;
    const TopoInfo *topo;
    const AlgEnvConfig *env;
    bool cuda;
    bool nvls;                 // multicast mapping exists
    uint64_t cclBytes;
    std::vector<HcclCommEngine> excluded;   // engines that already failed for this op (fallback path)
};

class AutoSelectorBase {
public:
    virtual ~AutoSelectorBase() = default;
    // Runs the engine cascade; fills param.engine / param.algName.
    SelectorStatus Select(const SelectorCtx &ctx, OpParam &param) const;
protected:
    virtual SelectorStatus SelectNvls(const SelectorCtx &, OpParam &) const { return SelectorStatus::NOT_MATCH; }
    virtual SelectorStatus SelectSm(const SelectorCtx &, OpParam &) const { return SelectorStatus::NOT_MATCH; }
    virtual SelectorStatus SelectIr(const SelectorCtx &, OpParam &) const { return SelectorStatus::NOT_MATCH; }  // HOST / COPY_ENGINE
    static bool IsSmallData(uint64_t bytes) { return bytes < (512u << 10); }     // reference: auto_selector_base.cc:82
    static bool IsLargeData(uint64_t bytes) { return bytes >= (1u << 20); }      // reference: auto_selector_base.cc:87
};

class SelectorRegistry {
public:
    static SelectorRegistry &Instance();
    void Register(HcclCMDType op, int priority, std::function<AutoSelectorBase *()> factory);
    // selectors for `op` by ascending priority value (lower runs first), instantiated once
    std::vector<AutoSelectorBase *> Get(HcclCMDType op);
private:
    struct Entry { int priority; std::function<AutoSelectorBase *()> factory; AutoSelectorBase *inst; };
    std::map<HcclCMDType, std::vector<Entry>> map_;
};

#define REGISTER_SELECTOR_BY_OPTYPE(op, priority, cls) \
    static bool g_sel_##cls##_##priority = (::hccl::SelectorRegistry::Instance().Register(op, priority, [] { return static_cast<::hccl::AutoSelectorBase *>(new cls()); }), true)

// Walks the registry for param.opType (MC2 ops use the priority-18 selector only, as in the reference).
HcclResult ExecuteSelector(const SelectorCtx &ctx, OpParam &param);

// ---- tuning table -------------------------------------------------------------------------------------------
struct TuningRow {
    uint64_t maxBytes;          // row applies to payloads <= maxBytes (rows sorted ascending; last row is the catch-all)
    std::string algName;
    uint32_t ctas;              // grid size hint (0 = default)
};
class TuningTable {
public:
    static TuningTable &Instance();
    // key: op, nranks (0 = any), engine
    const TuningRow *Lookup(HcclCMDType op, uint32_t nranks, HcclCommEngine engine, uint64_t bytes) const;
    void Set(HcclCMDType op, uint32_t nranks, HcclCommEngine engine, std::vector<TuningRow> rows);
    // text format, one row per line: "<op> <nranks> <engine> <maxBytes|inf> <algName> <ctas>"; '#' comments
    HcclResult LoadFile(const std::string &path);
    HcclResult LoadText(const std::string &text);
    void ResetToBuiltin();
    // Once per process: rows measured on the target machine that ship next to the library (<lib dir>/../tuning/b200.txt),
    // then the file named by HCCL_TUNING_FILE. Later rows replace earlier ones for the same (op, ranks, engine).
    HcclResult LoadConfigured(const std::string &envFile);
    std::string Dump() const;
private:
    TuningTable();
    struct Key { HcclCMDType op; uint32_t n; HcclCommEngine e; bool operator<(const Key &o) const { return std::tie(op, n, e) < std::tie(o.op, o.n, o.e); } };
    std::map<Key, std::vector<TuningRow>> rows_;
};

// Support matrices used by selectors and tests.
bool NvlsSupports(HcclDataType t, HcclReduceOp op);          // multimem.ld_reduce coverage
bool SmReduceSupports(HcclDataType t, HcclReduceOp op);      // in-kernel reduce coverage
const char *IrAlgoFor(HcclCMDType op, AlgoType forced, uint64_t bytes, uint32_t nranks, uint64_t cclBytes);

}  // namespace hccl
