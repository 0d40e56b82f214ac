// Algorithm templates that emit schedule IR (the host-issued engine; HCCL's "Ins*" AICPU template family,
// reference: src/ops/<op>/template/aicpu/*.cc, base class src/ops/op_common/template/alg_v2_template_base.h:18-76).
// A template works on a flat group of ranks (any level of the hierarchy) and on one chunk of the operator's data;
// the executor supplies buffer references, strides and the scratch window.
#pragma once
#include <functional>
#include <map>
#include <string>
#include <vector>
#include "plan.h"

namespace hccl {

// Notify slots (reference: alg_param.h:60-62 keeps ACK / DATA / FIN_ACK per channel)
enum : uint32_t { SLOT_ACK = 0, SLOT_DATA = 1, SLOT_FIN = 2, SLOT_READY = 3, SLOT_STEP_BASE = 4 };

struct TemplateCtx {
    std::vector<uint32_t> group;      // global ranks taking part, in template order
    uint32_t me = 0;                  // index of this rank in `group`
    uint32_t elemSize = 4;
    uint64_t count = 0;               // elements of this chunk (op-specific meaning, see OpParam::count)
    BufRef in, out;                   // chunk bases
    uint64_t inStride = 0, outStride = 0;   // bytes between per-rank blocks of the full user buffers
    uint64_t cclOff = 0, cclBytes = 0;      // scratch window inside the CCL half
    uint32_t root = 0;                // index in `group`
    bool inPlace = false;             // in and out alias
    // V variants, bytes, indexed by group position
    std::vector<uint64_t> sendBytes, sendOff, recvBytes, recvOff;
    uint32_t N() const { return (uint32_t)group.size(); }
};

struct IrTemplate {
    std::string name;
    HcclCMDType op;
    // bytes of scratch needed for `count` elements on n ranks
    std::function<uint64_t(const TemplateCtx &)> scratchBytes;
    // elements per chunk that fit into cclBytes (0 = unlimited / not chunkable)
    std::function<uint64_t(uint32_t n, uint32_t elemSize, uint64_t cclBytes)> maxCountPerLoop;
    std::function<HcclResult(const TemplateCtx &, Plan *)> gen;
    bool fullSyncEachCall;            // every rank synchronises with every other rank inside the plan
};

class IrTemplateRegistry {
public:
    static IrTemplateRegistry &Instance();
    void Register(const IrTemplate &t);
    const IrTemplate *Find(const std::string &name) const;
    std::vector<std::string> Names(HcclCMDType op) const;
private:
    std::map<std::string, IrTemplate> map_;
};

void RegisterBuiltinIrTemplates();   // idempotent

}  // namespace hccl
