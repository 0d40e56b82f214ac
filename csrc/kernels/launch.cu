// Host side of the SM / NVLS engine: plan an operator into launches, issue them on the caller's stream, and the
// single-GPU emulation harness used by the tests (all ranks on one device, one cooperative launch per chunk).
#include "../common/env_config.h"
#include <algorithm>
#include "../common/launch_count.h"
#include "launch.h"
#include <cuda_runtime.h>
#include <cstring>
#include "../common/dtype.h"
#include "../common/log.h"
#include "coll_args.h"
#include "emu_world.h"
#include "hccl/hccl_dfx.h"

namespace hccl {

thread_local std::vector<SmLaunch> *g_captureLaunches = nullptr;
HcclResult SmIssueEmuLaunch(const DevComm *devComms, int nranks, const SmLaunch &l0, const CollArgs *devArgs, const BatchArgs *devBatch,
                            cudaStream_t stream, bool pairKernel);

const std::vector<SmAlgoDesc> &SmAlgorithms()
{
    static const std::vector<SmAlgoDesc> v = {
        {"SmAllReduceMesh1DOneShot", HCCL_CMD_ALLREDUCE, false}, {"SmAllReduceMesh1DTwoShot", HCCL_CMD_ALLREDUCE, false},
        {"NvlsAllReduceOneShot", HCCL_CMD_ALLREDUCE, true}, {"NvlsAllReduceTwoShot", HCCL_CMD_ALLREDUCE, true},
        {"SmAllGatherMesh1D", HCCL_CMD_ALLGATHER, false}, {"SmAllGatherVMesh1D", HCCL_CMD_ALLGATHER_V, false},
        {"SmReduceScatterMesh1D", HCCL_CMD_REDUCE_SCATTER, false}, {"SmReduceScatterVMesh1D", HCCL_CMD_REDUCE_SCATTER_V, false},
        {"NvlsReduceScatter", HCCL_CMD_REDUCE_SCATTER, true},
        {"SmBroadcastMesh1D", HCCL_CMD_BROADCAST, false}, {"NvlsBroadcast", HCCL_CMD_BROADCAST, true},
        {"SmReduceMesh1D", HCCL_CMD_REDUCE, false}, {"SmScatterMesh1D", HCCL_CMD_SCATTER, false},
        {"SmAlltoAllMesh1D", HCCL_CMD_ALLTOALL, false}, {"SmAlltoAllVMesh1D", HCCL_CMD_ALLTOALLV, false},
        {"SmAlltoAllVCMesh1D", HCCL_CMD_ALLTOALLVC, false}, {"SmBarrierMesh1D", HCCL_CMD_BARRIER, false},
        {"SmAllReduceRing", HCCL_CMD_ALLREDUCE, false}, {"SmAllReduceConcurrent", HCCL_CMD_ALLREDUCE, false}, {"NvlsAllReduceConcurrent", HCCL_CMD_ALLREDUCE, true},
        {"SmAllReduceZeroCopy", HCCL_CMD_ALLREDUCE, false}, {"NvlsAllReduceZeroCopy", HCCL_CMD_ALLREDUCE, true},
        {"SmReduceScatterZeroCopy", HCCL_CMD_REDUCE_SCATTER, false}, {"NvlsReduceScatterZeroCopy", HCCL_CMD_REDUCE_SCATTER, true},
        {"SmAllGatherZeroCopy", HCCL_CMD_ALLGATHER, false}, {"NvlsAllGatherZeroCopy", HCCL_CMD_ALLGATHER, true},
        {"SmBroadcastZeroCopy", HCCL_CMD_BROADCAST, false}, {"NvlsBroadcastZeroCopy", HCCL_CMD_BROADCAST, true}, {"SmAllReducePipelined", HCCL_CMD_ALLREDUCE, false}, {"NvlsAllReducePipelined", HCCL_CMD_ALLREDUCE, true},
        {"SmReduceScatterPipelined", HCCL_CMD_REDUCE_SCATTER, false}, {"SmReduceScatterVPipelined", HCCL_CMD_REDUCE_SCATTER_V, false},
        {"NvlsReduceScatterPipelined", HCCL_CMD_REDUCE_SCATTER, true},
        {"SmAllGatherPush", HCCL_CMD_ALLGATHER, false}, {"SmAllGatherVPush", HCCL_CMD_ALLGATHER_V, false},
        {"NvlsAllGatherPush", HCCL_CMD_ALLGATHER, true}, {"NvlsAllGatherVPush", HCCL_CMD_ALLGATHER_V, true},
        {"SmBroadcastPush", HCCL_CMD_BROADCAST, false}, {"NvlsBroadcastPush", HCCL_CMD_BROADCAST, true},
        {"SmAlltoAllPush", HCCL_CMD_ALLTOALL, false},
        {"SmSend", HCCL_CMD_SEND, false}, {"SmRecv", HCCL_CMD_RECEIVE, false}, {"SmBatchSendRecv", HCCL_CMD_BATCH_SEND_RECV, false},
    };
    return v;
}

uint32_t SmDefaultCtas(HcclCMDType, const std::string &, uint64_t bytes, uint32_t) { return SmCtasFor(bytes, 0); }

HcclResult SmOrchestrate(Comm *c, OpParam &p, const std::string &algName)
{
    SmPlanCtx ctx;
    ctx.rank = c->rank;
    ctx.nranks = c->nranks;
    ctx.cclBytes = c->devComm.cclBytes;
    ctx.mailboxBytes = c->devComm.mailboxBytes;
    ctx.maxCtas = c->env.maxCtas;
    ctx.nvls = c->mcHeap != nullptr;
    ctx.registeredOffset = [c](const void *ptr, uint64_t bytes, uint64_t *off) { return CommRegisteredOffset(c, ptr, bytes, off); };
    if (c->env.multiDimSplitSet) { ctx.splitRatio[0] = c->env.multiDimSplitRatio[0]; ctx.splitRatio[1] = c->env.multiDimSplitRatio[1]; }
    std::vector<SmLaunch> launches;
    HcclResult r = SmPlanOp(ctx, p, algName, &launches);
    if (r != HCCL_SUCCESS) return r;
    for (const SmLaunch &l : launches) {
        HcclResult lr = SmIssueLaunch(c->devCommPtr, l, p.stream);
        if (lr != HCCL_SUCCESS) {
            HCCL_ERROR("launch of %s failed: %s", algName.c_str(), cudaGetErrorString(cudaGetLastError()));
            return lr;
        }
        c->counters.kernelsLaunched++;
        c->devOpIssued++;
        CountLaunch();
        c->counters.chunkLoops++;
    }
    if (g_captureLaunches) *g_captureLaunches = std::move(launches);
    return HCCL_SUCCESS;
}

}  // namespace hccl

using namespace hccl;

#define EMU_RT(call)                                                                              \
    do {                                                                                          \
        cudaError_t _e = (call);                                                                  \
        if (_e != cudaSuccess) { HCCL_ERROR("%s: %s", #call, cudaGetErrorString(_e)); return HCCL_E_RUNTIME; } \
    } while (0)

extern "C" {

HcclResult HcclEmuCreate(uint32_t nranks, uint64_t cclBytes, uint64_t arenaBytes, uint32_t waitTimeoutMs, void **emu)
{
    if (!emu || nranks == 0 || nranks > (uint32_t)kMaxRanks) return HCCL_E_PARA;
    auto *w = new EmuWorld();
    w->nranks = (int)nranks;
    w->cclBytes = (cclBytes + 127) & ~127ull;
    w->mailboxBytes = 256 << 10;
    uint64_t mailboxTotal = w->mailboxBytes * 2 * nranks;
    w->arenaOff = (kHeapHeaderBytes + 2 * w->cclBytes + mailboxTotal + 1023) & ~1023ull;
    w->arenaBytes = arenaBytes;
    uint64_t heapBytes = w->arenaOff + arenaBytes;
    EMU_RT(cudaHostAlloc((void **)&w->status, sizeof(DevStatus) * nranks, cudaHostAllocMapped));
    memset(w->status, 0, sizeof(DevStatus) * nranks);
    DevStatus *devStatus = nullptr;
    EMU_RT(cudaHostGetDevicePointer((void **)&devStatus, w->status, 0));
    w->heaps.resize(nranks);
    for (uint32_t r = 0; r < nranks; ++r) {
        EMU_RT(cudaMalloc((void **)&w->heaps[r], heapBytes));
        EMU_RT(cudaMemset(w->heaps[r], 0, kHeapHeaderBytes));
    }
    w->hostComms.resize(nranks);
    for (uint32_t r = 0; r < nranks; ++r) {
        DevComm &d = w->hostComms[r];
        memset(&d, 0, sizeof(d));
        d.rank = (int)r; d.nranks = (int)nranks; d.heapBytes = heapBytes;
        for (uint32_t q = 0; q < nranks; ++q) d.heap[q] = w->heaps[q];
        d.mcHeap = nullptr;
        d.cclOff[0] = kHeapHeaderBytes; d.cclOff[1] = kHeapHeaderBytes + w->cclBytes; d.cclBytes = w->cclBytes;
        d.mailboxOff = kHeapHeaderBytes + 2 * w->cclBytes; d.mailboxBytes = w->mailboxBytes;
        d.arenaOff = w->arenaOff; d.arenaBytes = w->arenaBytes;
        d.timeoutNs = (uint64_t)waitTimeoutMs * 1000000ull;
        d.status = devStatus + r;
        d.emuRanks = (int)nranks;
        d.traceOn = 1;
    }
    EMU_RT(cudaMalloc((void **)&w->devComms, sizeof(DevComm) * nranks));
    EMU_RT(cudaMemcpy(w->devComms, w->hostComms.data(), sizeof(DevComm) * nranks, cudaMemcpyHostToDevice));
    EMU_RT(cudaMalloc((void **)&w->devArgs, sizeof(CollArgs) * nranks));
    EMU_RT(cudaMalloc((void **)&w->devBatch, sizeof(BatchArgs) * nranks));
    EMU_RT(cudaMalloc(&w->devFusedParams, 2048 * nranks));
    EMU_RT(cudaDeviceSynchronize());
    *emu = w;
    return HCCL_SUCCESS;
}

HcclResult HcclEmuDestroy(void *emu)
{
    auto *w = (EmuWorld *)emu;
    if (!w) return HCCL_E_PTR;
    cudaDeviceSynchronize();
    for (char *h : w->heaps) cudaFree(h);
    cudaFree(w->devComms);
    cudaFree(w->devArgs);
    cudaFree(w->devBatch);
    cudaFree(w->devFusedParams);
    cudaFreeHost(w->status);
    delete w;
    return HCCL_SUCCESS;
}

// Runs one operator on all emulated ranks. ins/outs: per-rank device pointers. countMatrix: n*n elements for the
// AlltoAllV family (row i = what rank i sends), n elements for AllGatherV / ReduceScatterV, else unused.
HcclResult HcclEmuRun(void *emu, HcclCMDType op, const char *algName, void **ins, void **outs, uint64_t count, HcclDataType dataType,
                      HcclReduceOp reduceOp, uint32_t root, const uint64_t *countMatrix, uint32_t maxCtas)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !algName) return HCCL_E_PTR;
    uint32_t n = (uint32_t)w->nranks;
    std::vector<std::vector<SmLaunch>> per(n);
    for (uint32_t r = 0; r < n; ++r) {
        OpParam p;
        p.opType = op; p.inputPtr = ins ? ins[r] : nullptr; p.outputPtr = outs ? outs[r] : nullptr; p.count = count;
        p.dtype = p.outDtype = dataType; p.reduceOp = reduceOp; p.root = root;
        if (op == HCCL_CMD_ALLTOALLV || op == HCCL_CMD_ALLTOALLVC) {
            if (!countMatrix) return HCCL_E_PTR;
            p.sendCounts.resize(n); p.sendDispls.resize(n); p.recvCounts.resize(n); p.recvDispls.resize(n);
            uint64_t so = 0, ro = 0;
            for (uint32_t j = 0; j < n; ++j) {
                p.sendCounts[j] = countMatrix[r * n + j]; p.sendDispls[j] = so; so += p.sendCounts[j];
                p.recvCounts[j] = countMatrix[j * n + r]; p.recvDispls[j] = ro; ro += p.recvCounts[j];
            }
        } else if (op == HCCL_CMD_ALLGATHER_V || op == HCCL_CMD_REDUCE_SCATTER_V) {
            if (!countMatrix) return HCCL_E_PTR;
            auto &cnt = op == HCCL_CMD_ALLGATHER_V ? p.recvCounts : p.sendCounts;
            auto &dsp = op == HCCL_CMD_ALLGATHER_V ? p.recvDispls : p.sendDispls;
            cnt.assign(countMatrix, countMatrix + n);
            dsp.resize(n);
            uint64_t o = 0;
            for (uint32_t j = 0; j < n; ++j) { dsp[j] = o; o += cnt[j]; }
            p.count = cnt[r];
        }
        SmPlanCtx ctx{r, n, w->cclBytes, w->mailboxBytes, maxCtas ? maxCtas : 4u, false};
        (void)InitEnvConfig();
        // emulated ranks: a buffer inside a rank's arena counts as a registered window
        ctx.registeredOffset = [w, r](const void *ptr, uint64_t bytes, uint64_t *off) {
            const char *pc = (const char *)ptr, *base = w->heaps[r] + w->arenaOff;
            if (pc < base || pc + bytes > base + w->arenaBytes) return false;
            *off = (uint64_t)(pc - w->heaps[r]);
            return true;
        };
        if (GetEnvConfig().multiDimSplitSet) { ctx.splitRatio[0] = GetEnvConfig().multiDimSplitRatio[0]; ctx.splitRatio[1] = GetEnvConfig().multiDimSplitRatio[1]; }
        HcclResult pr = SmPlanOp(ctx, p, algName, &per[r]);
        if (pr != HCCL_SUCCESS) return pr;
    }
    for (uint32_t r = 1; r < n; ++r) {
        if (per[r].size() != per[0].size()) { HCCL_ERROR("emu: ranks disagree on the number of launches"); return HCCL_E_INTERNAL; }
    }
    for (size_t i = 0; i < per[0].size(); ++i) {
        std::vector<CollArgs> args(n);
        for (uint32_t r = 0; r < n; ++r) {
            if (per[r][i].kernel != per[0][i].kernel || per[r][i].ctas != per[0][i].ctas) { HCCL_ERROR("emu: ranks disagree on launch %zu", i); return HCCL_E_INTERNAL; }
            args[r] = per[r][i].args;
        }
        EMU_RT(cudaMemcpyAsync(w->devArgs, args.data(), sizeof(CollArgs) * n, cudaMemcpyHostToDevice, 0));
        HcclResult lr = SmIssueEmuLaunch(w->devComms, (int)n, per[0][i], w->devArgs, w->devBatch, 0, false);
        if (lr != HCCL_SUCCESS) { HCCL_ERROR("emu launch failed: %s", cudaGetErrorString(cudaGetLastError())); return lr; }
        EMU_RT(cudaStreamSynchronize(0));
    }
    for (uint32_t r = 0; r < n; ++r) if (w->status[r].code != 0) return HCCL_E_TIMEOUT;
    return HCCL_SUCCESS;
}

// Point-to-point in emulation: items[i] = {src, dst, srcBuf, dstBuf, bytes}; all transfers run in ONE launch through
// the batch kernel (each rank gets its own BatchArgs).
HcclResult HcclEmuBatchSendRecv(void *emu, uint32_t nTransfers, const uint32_t *srcRanks, const uint32_t *dstRanks, void **srcBufs,
                                void **dstBufs, const uint64_t *bytes)
{
    auto *w = (EmuWorld *)emu;
    if (!w) return HCCL_E_PTR;
    uint32_t n = (uint32_t)w->nranks;
    std::vector<SmLaunch> per(n);
    uint32_t maxCtas = 0;
    for (uint32_t r = 0; r < n; ++r) {
        OpParam p;
        p.opType = HCCL_CMD_BATCH_SEND_RECV;
        p.dtype = HCCL_DATA_TYPE_INT8;
        for (uint32_t t = 0; t < nTransfers; ++t) {
            if (srcRanks[t] == r) p.items.push_back(HcclSendRecvItem{HCCL_SEND, srcBufs[t], bytes[t], HCCL_DATA_TYPE_INT8, dstRanks[t]});
            if (dstRanks[t] == r) p.items.push_back(HcclSendRecvItem{HCCL_RECV, dstBufs[t], bytes[t], HCCL_DATA_TYPE_INT8, srcRanks[t]});
        }
        std::vector<SmLaunch> ls;
        SmPlanCtx ctx{r, n, w->cclBytes, w->mailboxBytes, 0, false};
        if (p.items.empty()) { SmLaunch l{}; l.kernel = K_BATCH_SEND_RECV; l.batch.nItems = 0; l.batch.nQueues = 0; l.ctas = kP2pBlocks; ls.push_back(l); }
        else { HcclResult pr = SmPlanOp(ctx, p, "SmBatchSendRecv", &ls); if (pr != HCCL_SUCCESS) return pr; }
        per[r] = ls[0];
        maxCtas = std::max(maxCtas, per[r].ctas);
    }
    std::vector<BatchArgs> b(n);
    for (uint32_t r = 0; r < n; ++r) b[r] = per[r].batch;
    EMU_RT(cudaMemcpyAsync(w->devBatch, b.data(), sizeof(BatchArgs) * n, cudaMemcpyHostToDevice, 0));
    SmLaunch l0 = per[0];
    l0.ctas = maxCtas;
    HcclResult lr = SmIssueEmuLaunch(w->devComms, (int)n, l0, w->devArgs, w->devBatch, 0, false);
    if (lr != HCCL_SUCCESS) { HCCL_ERROR("emu batch launch failed: %s", cudaGetErrorString(cudaGetLastError())); return lr; }
    EMU_RT(cudaStreamSynchronize(0));
    for (uint32_t r = 0; r < n; ++r) if (w->status[r].code != 0) return HCCL_E_TIMEOUT;
    return HCCL_SUCCESS;
}

// Reads (and optionally clears) the status word of an emulated rank: out[0..7] = DevStatus fields.
HcclResult HcclEmuStatus(void *emu, uint32_t rank, uint32_t *out, int clear)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !out || rank >= (uint32_t)w->nranks) return HCCL_E_PARA;
    memcpy(out, &w->status[rank], sizeof(DevStatus));
    if (clear) {
        memset(&w->status[rank], 0, sizeof(DevStatus));
        for (char *h : w->heaps) cudaMemset(h, 0, kHeapHeaderBytes);
        cudaDeviceSynchronize();
    }
    return HCCL_SUCCESS;
}

// Base address and size of an emulated rank's arena (the part of its heap that stands for symmetric user allocations).
HcclResult HcclEmuArena(void *emu, uint32_t rank, void **base, uint64_t *bytes)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !base || !bytes || rank >= (uint32_t)w->nranks) return HCCL_E_PARA;
    *base = w->heaps[rank] + w->arenaOff;
    *bytes = w->arenaBytes;
    return HCCL_SUCCESS;
}

// Device-side trace of an emulated rank: up to maxRecords rows {seq, syncs, enterNs, firstSyncNs, lastSyncNs, leaveNs}, oldest first.
HcclResult HcclEmuTrace(void *emu, uint32_t rank, uint64_t *rows, uint32_t maxRecords, uint32_t *numRecords)
{
    auto *w = (EmuWorld *)emu;
    if (!w || !rows || !numRecords || rank >= (uint32_t)w->nranks) return HCCL_E_PARA;
    std::vector<uint8_t> ctrl(sizeof(DevCtrl));
    EMU_RT(cudaMemcpy(ctrl.data(), w->heaps[rank], ctrl.size(), cudaMemcpyDeviceToHost));
    const DevCtrl *dc = reinterpret_cast<const DevCtrl *>(ctrl.data());
    std::vector<DevTraceRec> recs;
    for (int i = 0; i < kTraceSlots; ++i) if (dc->trace[i].tEnter != 0) recs.push_back(dc->trace[i]);
    std::sort(recs.begin(), recs.end(), [](const DevTraceRec &a, const DevTraceRec &b) { return a.seq < b.seq; });
    *numRecords = 0;
    for (size_t i = recs.size() > maxRecords ? recs.size() - maxRecords : 0; i < recs.size(); ++i) {
        uint64_t *r = rows + 6 * (*numRecords)++;
        r[0] = recs[i].seq; r[1] = recs[i].barriers; r[2] = recs[i].tEnter; r[3] = recs[i].tBarrier[0]; r[4] = recs[i].tBarrier[1]; r[5] = recs[i].tLeave;
    }
    return HCCL_SUCCESS;
}

// Test hook for the bounded wait: launches the barrier kernel for ONE emulated rank only, so its peers never
// signal; the kernel must give up after the timeout, set the status word and return.
HcclResult HcclEmuLonelyBarrier(void *emu, uint32_t rank)
{
    auto *w = (EmuWorld *)emu;
    if (!w || rank >= (uint32_t)w->nranks) return HCCL_E_PARA;
    SmLaunch l{};
    l.kernel = K_BARRIER;
    l.ctas = 1;
    HcclResult lr = SmIssueLaunch(w->devComms + rank, l, 0);
    if (lr != HCCL_SUCCESS) return lr;
    EMU_RT(cudaStreamSynchronize(0));
    return w->status[rank].code == 1 ? HCCL_E_TIMEOUT : HCCL_SUCCESS;
}

}  // extern "C"
