// MC2 argument blob and resource-context API (reference: include/hccl_mc2.h:25-82; src/common/hccl_mc2.cc:21-36 HcclOpArgs
// with defaults fp16 / sum / 0, :117 algConfig limited to 128 characters, :130-133 engine restricted to the device-side
// engines, :141-165 HcclCreateOpResCtx validates and forwards to the communicator layer). The context handed back is a
// device-resident description of the symmetric heap that a caller's own fused kernel can use to reach its peers.
#include <cstring>
#include "../common/dtype.h"
#include "../common/env_config.h"
#include "../common/log.h"
#include "../common/param_check.h"
#include "../core/comm.h"
#include "hccl/hccl_mc2.h"

using namespace hccl;

namespace hccl {
HcclResult CudaMemsetDevice(void *dst, int v, uint64_t bytes);
}

namespace {
constexpr uint32_t kArgsMagic = 0x4b464341u;   // 'KFCA'
struct HcclOpArgs {
    uint32_t magic = kArgsMagic;
    uint8_t srcDataType = HCCL_DATA_TYPE_FP16;
    uint8_t dstDataType = HCCL_DATA_TYPE_FP16;
    uint32_t reduceType = HCCL_REDUCE_SUM;
    uint64_t count = 0;
    char algConfig[ALG_CONFIG_MAX_LEN] = {0};
    uint8_t commEngine = HCCL_ENGINE_SM;
};
HcclOpArgs *Args(void *p)
{
    auto *a = static_cast<HcclOpArgs *>(p);
    return (a && a->magic == kArgsMagic) ? a : nullptr;
}
}  // namespace

extern "C" {

HcclResult HcclKfcAllocOpArgs(void **opArgs)
{
    CHK_PTR_NULL(opArgs);
    *opArgs = new (std::nothrow) HcclOpArgs();
    return *opArgs ? HCCL_SUCCESS : HCCL_E_MEMORY;
}
HcclResult HcclKfcFreeOpArgs(void *opArgs)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] HcclKfcFreeOpArgs: not an op-args blob"), HCCL_E_PTR);
    a->magic = 0;
    delete a;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetSrcDataType(void *opArgs, uint8_t srcDataType)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] op args is null or corrupt"), HCCL_E_PTR);
    CHK_RET(HcomCheckDataType((HcclDataType)srcDataType));
    a->srcDataType = srcDataType;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetDstDataType(void *opArgs, uint8_t dstDataType)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] op args is null or corrupt"), HCCL_E_PTR);
    CHK_RET(HcomCheckDataType((HcclDataType)dstDataType));
    a->dstDataType = dstDataType;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetReduceType(void *opArgs, uint32_t reduceType)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] op args is null or corrupt"), HCCL_E_PTR);
    CHK_RET(HcomCheckReductionOp((HcclReduceOp)reduceType));
    a->reduceType = reduceType;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetCount(void *opArgs, uint64_t count)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] op args is null or corrupt"), HCCL_E_PTR);
    CHK_RET(HcomCheckCount(count));
    a->count = count;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetAlgConfig(void *opArgs, char *algConfig)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] op args is null or corrupt"), HCCL_E_PTR);
    CHK_PTR_NULL(algConfig);
    size_t n = strnlen(algConfig, ALG_CONFIG_MAX_LEN);
    CHK_PRT_RET(n >= ALG_CONFIG_MAX_LEN, HCCL_ERROR("[EI0003] algConfig is longer than %u characters", ALG_CONFIG_MAX_LEN - 1), HCCL_E_PARA);
    memset(a->algConfig, 0, sizeof(a->algConfig));
    memcpy(a->algConfig, algConfig, n);
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetCommEngine(void *opArgs, uint8_t commEngine)
{
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] op args is null or corrupt"), HCCL_E_PTR);
    CHK_PRT_RET(commEngine != HCCL_ENGINE_SM && commEngine != HCCL_ENGINE_NVLS,
                HCCL_ERROR("[EI0003] commEngine %u: a fused kernel can only use the device-side engines SM (%d) or NVLS (%d)", commEngine, HCCL_ENGINE_SM, HCCL_ENGINE_NVLS),
                HCCL_E_PARA);
    a->commEngine = commEngine;
    return HCCL_SUCCESS;
}

// Reserves a window of the symmetric arena (count * sizeof(dst) * ranks bytes + 64 KB of zeroed flag words), writes the
// HcclOpResCtx description into device memory and returns its device address. One context per (opType, algConfig) key.
HcclResult HcclCreateOpResCtx(HcclComm comm, uint8_t opType, void *opArgs, void **opResCtx)
{
    CHK_RET(InitEnvConfig());
    Comm *c = CommFromHandle(comm);
    CHK_PRT_RET(!c, HCCL_ERROR("[EI0003] HcclCreateOpResCtx: comm is not a live communicator"), HCCL_E_PTR);
    HcclOpArgs *a = Args(opArgs);
    CHK_PRT_RET(!a, HCCL_ERROR("[EI0003] HcclCreateOpResCtx: op args is null or corrupt"), HCCL_E_PTR);
    CHK_PTR_NULL(opResCtx);
    CHK_PRT_RET(opType == HCCL_CMD_INVALID || opType >= HCCL_CMD_MAX, HCCL_ERROR("[EI0003] HcclCreateOpResCtx: opType %u is invalid", opType), HCCL_E_PARA);
    CHK_PRT_RET(a->commEngine == HCCL_ENGINE_NVLS && c->mcHeap == nullptr,
                HCCL_ERROR("HcclCreateOpResCtx: NVLS engine requested but the communicator has no multicast mapping"), HCCL_E_UNAVAIL);
    if (c->env.entryLogEnable)
        HCCL_RUN_INFO("Entry-HcclCreateOpResCtx: opType[%u] src[%s] dst[%s] reduce[%s] count[%llu] algConfig[%s] engine[%u]", opType,
                      DataTypeName((HcclDataType)a->srcDataType), DataTypeName((HcclDataType)a->dstDataType), ReduceOpName((HcclReduceOp)a->reduceType),
                      (unsigned long long)a->count, a->algConfig, a->commEngine);
    const std::string tag = std::string("mc2ctx_") + CmdName((HcclCMDType)opType) + "_" + a->algConfig;
    void *existing = nullptr;
    uint64_t bytes = 0;
    if (EngineCtxGet(c, tag, c->backend == BackendKind::CUDA, &existing, &bytes) == HCCL_SUCCESS) { *opResCtx = existing; return HCCL_SUCCESS; }
    const uint64_t flagBytes = 64 << 10;
    uint64_t payload = a->count * DataTypeSize((HcclDataType)a->dstDataType) * c->nranks;
    uint64_t wsBytes = ((payload + 255) & ~255ull) + flagBytes;
    void *ws = nullptr;
    CHK_RET(SymAlloc(c, wsBytes, &ws));
    HcclOpResCtx ctx;
    memset(&ctx, 0, sizeof(ctx));
    ctx.magic = 0x4332434du;   // 'MC2C'
    ctx.opType = opType;
    ctx.rank = c->rank;
    ctx.nranks = c->nranks;
    ctx.srcDataType = a->srcDataType; ctx.dstDataType = a->dstDataType; ctx.reduceType = a->reduceType; ctx.commEngine = a->commEngine;
    ctx.count = a->count;
    ctx.heapBytes = c->heapBytes;
    for (uint32_t r = 0; r < c->nranks; ++r) ctx.heap[r] = c->heap[r];
    ctx.mcHeap = c->mcHeap;
    ctx.workspaceOff = SymOffsetOf(c, ws);
    ctx.workspaceBytes = wsBytes;
    ctx.flagOff = ctx.workspaceOff + wsBytes - flagBytes;
    ctx.timeoutNs = c->devComm.timeoutNs;
    memcpy(ctx.algConfig, a->algConfig, sizeof(ctx.algConfig));
    const bool onDevice = c->backend == BackendKind::CUDA;
    void *blob = nullptr;
    CHK_RET(EngineCtxCreate(c, tag, onDevice, sizeof(ctx), &blob));
    if (onDevice) {
        CHK_RET(EngineCtxCopy(c, tag, &ctx, sizeof(ctx)));
        CHK_RET(CudaMemsetDevice((char *)ws + wsBytes - flagBytes, 0, flagBytes));
    } else {
        memcpy(blob, &ctx, sizeof(ctx));
        memset((char *)ws + wsBytes - flagBytes, 0, flagBytes);
    }
    // every rank has zeroed its flags before any peer may touch them
    CHK_RET(c->boot->Barrier());
    *opResCtx = blob;
    return HCCL_SUCCESS;
}

}  // extern "C"
