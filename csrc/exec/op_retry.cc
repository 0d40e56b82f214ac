// Operator retry: after a wait timeout, re-run the operator every rank stopped at.
//
// HCCL re-executes a failed operator when (a) retry is switched on for the communicator's scope, (b) all ranks stopped at
// the same operator and (c) the operator's input cannot have been overwritten (not in place, no zero-copy reduction);
// hosts agree over their sockets, then the operator is issued again from its input, up to MaxCnt times, and
// HCCL_E_OPRETRY_FAIL is returned when that does not help (reference: docs/zh/user_guide/hccl_env/HCCL_OP_RETRY_ENABLE.md:5-60,
// HCCL_OP_RETRY_PARAMS.md, src/common/alg_env_config.cc:914). Here:
//   1. every operator call leaves a copy of its parameters in the communicator;
//   2. a rank whose wait ran out (device status record or host-engine timeout), or that learnt of a peer's timeout through
//      the heartbeat, finds the communicator suspended at its next call and enters CommOpRetry;
//   3. the ranks all-gather (operator index, input intact?) over the bootstrap; any disagreement ends the retry;
//   4. per attempt: wait (HoldTime first, IntervalTime between attempts), resume the communicator on all ranks (flags and
//      status cleared between two barriers), issue the recorded operator again, wait for it, all-gather the outcome.
// The failing call is made on the host in the tests (a rank that records an operator but does not launch it); nothing
// here needs, or causes, a device fault.
#include <chrono>
#include <cstring>
#include <thread>
#include "../common/dtype.h"
#include "../common/log.h"
#include "op_common.h"

namespace hccl {

extern HcclResult CudaStreamSync(cudaStream_t s);

bool OpRetryEnabled(const Comm *c) { return c->env.opRetryIntraServer || c->env.opRetryInterServer || c->env.opRetryInterSuperPod; }

namespace {
bool InputIntact(const OpParam &p)
{
    switch (p.opType) {
        case HCCL_CMD_BROADCAST: return true;                      // every rank but the root only receives; the root's buffer is never written
        case HCCL_CMD_BARRIER: return true;
        case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: case HCCL_CMD_BATCH_SEND_RECV: return false;   // pairwise: the group cannot agree on them
        default: return p.inputPtr != nullptr && p.inputPtr != p.outputPtr;
    }
}
struct Vote { uint64_t seq; uint32_t intact, opType; };
struct Outcome { uint32_t ok; };

HcclResult WaitIssued(Comm *c, cudaStream_t s)
{
    if (c->backend == BackendKind::SIM) return c->worker ? c->worker->Drain() : HCCL_SUCCESS;
    HcclResult r = CudaStreamSync(s);
    if (r != HCCL_SUCCESS) return r;
    return (c->hostStatus && c->hostStatus->code != 0) ? HCCL_E_TIMEOUT : HCCL_SUCCESS;
}
}  // namespace

void RecordOpForRetry(Comm *c, const OpParam &p)
{
    std::lock_guard<std::mutex> lk(c->retryMu);
    c->retryOp = std::make_shared<OpParam>(p);
    c->retrySeq = c->counters.ops.load();
    c->retryInputIntact = InputIntact(p);
}

HcclResult CommOpRetry(Comm *c)
{
    struct Guard {
        Comm *c;
        explicit Guard(Comm *cc) : c(cc) { c->inRetry = true; }
        ~Guard() { c->inRetry = false; }
    } guard(c);
    std::shared_ptr<OpParam> op;
    Vote mine{};
    {
        std::lock_guard<std::mutex> lk(c->retryMu);
        op = std::static_pointer_cast<OpParam>(c->retryOp);
        mine.seq = c->retrySeq;
        mine.intact = op && c->retryInputIntact ? 1u : 0u;
        mine.opType = op ? (uint32_t)op->opType : 0u;
    }
    // nothing of this rank may still be running when the group decides
    if (c->worker) (void)c->worker->Drain();
    if (c->backend == BackendKind::CUDA) (void)CudaBackendQuiesce(c);
    std::vector<Vote> votes(c->nranks);
    CHK_RET(c->boot->AllGather(&mine, sizeof(mine), votes.data()));
    for (uint32_t r = 0; r < c->nranks; ++r) {
        if (votes[r].seq != mine.seq || votes[r].opType != mine.opType) {
            HCCL_ERROR("operator retry on comm %s: rank %u stopped at operator %llu (%s), rank %u at %llu (%s); the ranks are not at the same operator",
                       c->name.c_str(), c->rank, (unsigned long long)mine.seq, CmdName((HcclCMDType)mine.opType), r, (unsigned long long)votes[r].seq,
                       CmdName((HcclCMDType)votes[r].opType));
            return HCCL_E_OPRETRY_FAIL;
        }
        if (!votes[r].intact) {
            HCCL_ERROR("operator retry on comm %s: the input of operator %llu (%s) on rank %u may have been overwritten (in place, or not recorded)",
                       c->name.c_str(), (unsigned long long)mine.seq, CmdName((HcclCMDType)mine.opType), r);
            return HCCL_E_OPRETRY_FAIL;
        }
    }
    const uint32_t maxCnt = c->env.opRetryMaxCnt ? c->env.opRetryMaxCnt : 1;
    for (uint32_t attempt = 1; attempt <= maxCnt; ++attempt) {
        std::this_thread::sleep_for(std::chrono::milliseconds(attempt == 1 ? c->env.opRetryHoldTimeMs : c->env.opRetryIntervalMs));
        HCCL_RUN_INFO("comm %s rank %u: retrying operator %llu (%s), attempt %u of %u", c->name.c_str(), c->rank, (unsigned long long)mine.seq,
                      CmdName(op->opType), attempt, maxCnt);
        CHK_RET(CommResume(c));
        c->counters.opRetries++;
        OpParam again = *op;
        HcclResult r = HcclExecOp(c, again);
        if (r == HCCL_SUCCESS) r = WaitIssued(c, again.stream);
        Outcome me{r == HCCL_SUCCESS ? 1u : 0u};
        std::vector<Outcome> all(c->nranks);
        CHK_RET(c->boot->AllGather(&me, sizeof(me), all.data()));
        bool ok = true;
        for (auto &o : all) ok = ok && o.ok;
        if (ok) {
            HCCL_RUN_INFO("comm %s rank %u: operator %llu completed on attempt %u", c->name.c_str(), c->rank, (unsigned long long)mine.seq, attempt);
            return HCCL_SUCCESS;
        }
        if (r == HCCL_SUCCESS) CommSuspend(c);     // a peer failed again: stay out of the next operator until the next attempt resumes everyone
        else CommPollAsyncError(c, nullptr);
    }
    HCCL_ERROR("operator retry on comm %s rank %u: operator %llu (%s) still fails after %u attempts", c->name.c_str(), c->rank,
               (unsigned long long)mine.seq, CmdName(op->opType), maxCnt);
    return HCCL_E_OPRETRY_FAIL;
}

}  // namespace hccl
