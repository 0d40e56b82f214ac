#include "host_engine.h"
#include <chrono>
#include <cstring>
#include <thread>
#include "../common/dtype.h"
#include "../common/log.h"

namespace hccl {
namespace {

template <typename T> inline T ApplyOp(T a, T b, HcclReduceOp op)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return (T)(a + b);
        case HCCL_REDUCE_PROD: return (T)(a * b);
        case HCCL_REDUCE_MAX: return a > b ? a : b;
        case HCCL_REDUCE_MIN: return a < b ? a : b;
        default: return a;
    }
}
template <typename T> void ReduceTyped(void *dst, const void *src, uint64_t n, HcclReduceOp op)
{
    T *d = (T *)dst;
    const T *s = (const T *)src;
    for (uint64_t i = 0; i < n; ++i) d[i] = ApplyOp<T>(d[i], s[i], op);
}
template <float (*ToF)(uint16_t), uint16_t (*FromF)(float)> void ReduceHalf(void *dst, const void *src, uint64_t n, HcclReduceOp op)
{
    uint16_t *d = (uint16_t *)dst;
    const uint16_t *s = (const uint16_t *)src;
    for (uint64_t i = 0; i < n; ++i) d[i] = FromF(ApplyOp<float>(ToF(d[i]), ToF(s[i]), op));
}

int64_t NowMs()
{
    using namespace std::chrono;
    return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

}  // namespace

HcclResult HostReduce(void *dst, const void *src, uint64_t bytes, HcclDataType dtype, HcclReduceOp op)
{
    uint32_t es = DataTypeSize(dtype);
    if (es == 0 || bytes % es) return HCCL_E_PARA;
    uint64_t n = bytes / es;
    switch (dtype) {
        case HCCL_DATA_TYPE_INT8: ReduceTyped<int8_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_INT16: ReduceTyped<int16_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_INT32: ReduceTyped<int32_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_INT64: ReduceTyped<int64_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_UINT64: ReduceTyped<uint64_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_UINT8: ReduceTyped<uint8_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_UINT16: ReduceTyped<uint16_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_UINT32: ReduceTyped<uint32_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_FP32: ReduceTyped<float>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_FP64: ReduceTyped<double>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_FP16: ReduceHalf<Fp16ToFloat, FloatToFp16>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_BFP16: ReduceHalf<Bf16ToFloat, FloatToBf16>(dst, src, n, op); break;
        default: return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

HcclResult HostEngineRun(Comm *c, const Plan &plan, const ExecBuffers &bufs)
{
    const DevComm &d = c->devComm;
    DevCtrl *ctrl = CtrlOf(c->heap[c->rank]);
    DevFlags *myFlags = FlagsOf(c->heap[c->rank]);
    auto local = [&](const BufRef &b) -> char * {
        switch (b.kind) {
            case BufKind::INPUT: return bufs.in + b.off;
            case BufKind::OUTPUT: return bufs.out + b.off;
            case BufKind::CCL: return c->heap[c->rank] + d.cclOff[bufs.cclHalf] + b.off;
            case BufKind::MAILBOX: return c->heap[c->rank] + d.mailboxOff + b.off;
            case BufKind::ABS: return reinterpret_cast<char *>(b.off);
        }
        return nullptr;
    };
    auto remote = [&](uint32_t rank, const BufRef &b) -> char * {
        uint64_t base = b.kind == BufKind::MAILBOX ? d.mailboxOff : d.cclOff[bufs.cclHalf];
        return c->heap[rank] + base + b.off;
    };
    auto inBounds = [&](const BufRef &b, uint64_t bytes) {
        if (b.kind == BufKind::CCL) return b.off + bytes <= d.cclBytes;
        if (b.kind == BufKind::MAILBOX) return b.off + bytes <= d.mailboxBytes * 2 * (uint64_t)d.nranks;
        return true;
    };

    size_t nq = plan.queues.size();
    std::vector<size_t> pc(nq, 0);
    std::vector<std::vector<uint64_t>> localSem(nq, std::vector<uint64_t>(nq, 0)), localWaited(nq, std::vector<uint64_t>(nq, 0));
    int64_t lastProgress = NowMs();
    const int64_t timeoutMs = (int64_t)c->env.deviceWaitTimeoutMs;
    size_t done = 0;
    for (auto &q : plan.queues) if (q.empty()) ++done;
    uint32_t spins = 0;
    while (done < nq) {
        bool progressed = false;
        for (size_t qi = 0; qi < nq; ++qi) {
            const auto &q = plan.queues[qi];
            while (pc[qi] < q.size()) {
                const Task &t = q[pc[qi]];
                bool blocked = false;
                switch (t.type) {
                    case TaskType::LOCAL_COPY:
                        if (!inBounds(t.dst, t.bytes) || !inBounds(t.src, t.bytes)) return HCCL_E_INTERNAL;
                        if (local(t.dst) != local(t.src)) memmove(local(t.dst), local(t.src), t.bytes);
                        break;
                    case TaskType::LOCAL_REDUCE:
                        if (!inBounds(t.dst, t.bytes) || !inBounds(t.src, t.bytes)) return HCCL_E_INTERNAL;
                        CHK_RET(HostReduce(local(t.dst), local(t.src), t.bytes, plan.dtype, plan.op));
                        break;
                    case TaskType::WRITE:
                        if (!inBounds(t.dst, t.bytes)) return HCCL_E_INTERNAL;
                        memcpy(remote(t.rank, t.dst), local(t.src), t.bytes);
                        break;
                    case TaskType::WRITE_REDUCE:
                        if (!inBounds(t.dst, t.bytes)) return HCCL_E_INTERNAL;
                        CHK_RET(HostReduce(remote(t.rank, t.dst), local(t.src), t.bytes, plan.dtype, plan.op));
                        break;
                    case TaskType::READ:
                        if (!inBounds(t.src, t.bytes)) return HCCL_E_INTERNAL;
                        memcpy(local(t.dst), remote(t.rank, t.src), t.bytes);
                        break;
                    case TaskType::READ_REDUCE:
                        if (!inBounds(t.src, t.bytes)) return HCCL_E_INTERNAL;
                        CHK_RET(HostReduce(local(t.dst), remote(t.rank, t.src), t.bytes, plan.dtype, plan.op));
                        break;
                    case TaskType::POST: {
                        if (t.slot >= (uint32_t)kNotifySlots) return HCCL_E_INTERNAL;
                        uint64_t v = ++ctrl->hostNotifySent[t.rank][t.slot];
                        __atomic_store_n(&FlagsOf(c->heap[t.rank])->hostNotify[c->rank][t.slot], v, __ATOMIC_RELEASE);
                        break;
                    }
                    case TaskType::WAIT: {
                        if (t.slot >= (uint32_t)kNotifySlots) return HCCL_E_INTERNAL;
                        uint64_t want = ctrl->hostNotifyWaited[t.rank][t.slot] + 1;
                        uint64_t have = __atomic_load_n(&myFlags->hostNotify[t.rank][t.slot], __ATOMIC_ACQUIRE);
                        if (have >= want) ctrl->hostNotifyWaited[t.rank][t.slot] = want;
                        else blocked = true;
                        break;
                    }
                    case TaskType::LOCAL_POST:
                        if (t.rank >= nq) return HCCL_E_INTERNAL;
                        localSem[t.rank][qi]++;
                        break;
                    case TaskType::LOCAL_WAIT:
                        if (t.rank >= nq) return HCCL_E_INTERNAL;
                        if (localSem[qi][t.rank] > localWaited[qi][t.rank]) localWaited[qi][t.rank]++;
                        else blocked = true;
                        break;
                }
                if (blocked) break;
                ++pc[qi];
                progressed = true;
                if (pc[qi] == q.size()) ++done;
            }
        }
        if (progressed) { lastProgress = NowMs(); spins = 0; continue; }
        if (c->status.load() != HCCL_COMM_STATUS_READY) return HCCL_E_SUSPENDING;
        if (++spins > 64) { std::this_thread::yield(); }
        if ((spins & 0x3ff) == 0 && NowMs() - lastProgress > timeoutMs) {
            // report the first blocked wait
            for (size_t qi = 0; qi < nq; ++qi) {
                if (pc[qi] >= plan.queues[qi].size()) continue;
                const Task &t = plan.queues[qi][pc[qi]];
                if (t.type != TaskType::WAIT) continue;
                DevStatus &s = *c->hostStatus;
                s.rank = c->rank; s.peer = t.rank; s.channel = (uint32_t)qi; s.phase = t.slot; s.opSeq = (uint32_t)c->opSeq;
                s.observed = (uint32_t)myFlags->hostNotify[t.rank][t.slot];
                s.expected = (uint32_t)(ctrl->hostNotifyWaited[t.rank][t.slot] + 1);
                __atomic_store_n(&s.code, 1u, __ATOMIC_RELEASE);
                HCCL_ERROR("host engine: rank %u timed out after %lld ms waiting for rank %u slot %u (task %zu of queue %zu)", c->rank,
                           (long long)timeoutMs, t.rank, t.slot, pc[qi], qi);
                break;
            }
            return HCCL_E_TIMEOUT;
        }
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
