// Shared helpers of the operator entry points (argument checks -> OpParam -> dispatch core).
// The per-op flow mirrors HCCL's entries (reference: src/ops/all_reduce/all_reduce_op.cc:23-56,106-178): env init,
// zero-count shortcut, null / rank / count / dtype / op checks with EI0003 reporting, tag "<Op>_<commName>",
// fill OpParam, hand over to HcclExecOp.
#pragma once
#include <string>
#include "../common/dtype.h"
#include "../common/env_config.h"
#include "../common/log.h"
#include "../common/param_check.h"
#include "../core/comm.h"
#include "../exec/op_common.h"
#include "../exec/op_param.h"

namespace hccl {

inline HcclResult EntryCommon(HcclComm comm, Comm **out)
{
    CHK_RET(InitEnvConfig());
    if (comm == nullptr) { HCCL_ERROR("[EI0003] comm is null"); return HCCL_E_PTR; }
    Comm *c = CommFromHandle(comm);
    if (c == nullptr) { HCCL_ERROR("[EI0003] comm %p is not a live communicator", comm); return HCCL_E_PARA; }
    *out = c;
    return HCCL_SUCCESS;
}

inline OpParam MakeParam(Comm *c, HcclCMDType op, const char *name, cudaStream_t stream)
{
    OpParam p;
    p.opType = op;
    p.tag = std::string(name) + "_" + c->name;
    p.stream = stream;
    return p;
}

// Guards every entry point: exceptions never cross the C ABI.
template <typename F> HcclResult Guard(const char *what, F &&f)
{
    try {
        return f();
    } catch (const std::exception &e) {
        HCCL_ERROR("%s: unexpected exception: %s", what, e.what());
        return HCCL_E_INTERNAL;
    } catch (...) {
        HCCL_ERROR("%s: unexpected exception", what);
        return HCCL_E_INTERNAL;
    }
}

}  // namespace hccl
