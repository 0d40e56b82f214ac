// What the library does when a device-side (or host-engine) wait runs out, and how it notices that nothing moves.
//
//   * Task-exception dump: the first time a communicator sees a status record with a non-zero code it copies its control
//     block and flag arena to the host, names the flag words of the failing channel that are behind, and lists the last
//     operators. With HCCL_EXCEPTION_DUMP_DIR set the same data is written as a binary file that HcclReadExceptionDump
//     turns back into text. (HCCL dumps the flag memory and the last 50 tasks when a vector-core kernel reports an
//     exception; reference: src/ops/op_common/template/aiv/hccl_aiv_utils.cc:266-310.)
//   * Progress counters for the heartbeat: operators issued / completed on this rank, so that the watchdog can tell a
//     stuck communicator from an idle one and name the slowest rank (reference: the STUCK heartbeat state,
//     docs/zh/user_guide/fault_diagnosis/task_exec_stage.md:18-28).
// Nothing here touches a kernel in flight: the copies run on a private stream after the reporting kernel has returned.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include "../common/binary_stream.h"
#include "../common/dtype.h"
#include "../common/log.h"
#include "../core/comm.h"
#include "hccl/hccl_dfx.h"

namespace hccl {

namespace {
constexpr uint32_t kDumpMagic = 0x58454348u;   // 'HCEX'
constexpr uint32_t kDumpVersion = 1;

struct OpRecordPod {    // trivially copyable mirror of OpRecord for the dump file
    uint64_t seq; uint32_t opType, dtype, reduceOp, root, engine, pad; uint64_t count; char algName[64]; uint64_t beginNs, endNs;
};

std::string DescribeFlags(const DevStatus &s, const DevCtrl *ctrl, const DevFlags *flags, uint32_t nranks)
{
    std::ostringstream o;
    o << "opCount=" << ctrl->opCount << " abortFlag=" << ctrl->abortFlag;
    const uint32_t ch = s.channel;
    if (ch < (uint32_t)kMaxChannels) {
        o << " channel " << ch << " epoch=" << ctrl->chanEpoch[ch] << " barrier flags by source rank:";
        for (uint32_t r = 0; r < nranks && r < (uint32_t)kMaxRanks; ++r) {
            o << " r" << r << "=" << flags->barrier[ch][r];
            if ((int32_t)(flags->barrier[ch][r] - s.expected) < 0 && s.phase < 30) o << "(behind)";
        }
        o << "; chunk flags:";
        for (uint32_t r = 0; r < nranks && r < (uint32_t)kMaxRanks; ++r) o << " r" << r << "=" << flags->chunk[ch][r];
    }
    o << "; host notifies from rank " << s.peer << ":";
    if (s.peer < (uint32_t)kMaxRanks)
        for (int k = 0; k < 4; ++k) o << " s" << k << "=" << flags->hostNotify[s.peer][k];
    return o.str();
}
}  // namespace

void CommProgress(Comm *c, uint64_t *issued, uint64_t *done)
{
    if (c->backend == BackendKind::SIM) {
        *issued = c->worker ? c->worker->Enqueued() : 0;
        *done = c->worker ? c->worker->Completed() : 0;
        return;
    }
    // CUDA: kernels issued by the host against kernels that have been entered on the device (the op counter in the
    // control block advances once per collective kernel). Fused and MoE kernels advance it as well.
    // The last CTA to enter a kernel mirrors the counter into a pinned host word, so the watchdog thread reads plain memory
    // and never calls into the CUDA runtime. The device counter is 32 bits wide: compare modulo 2^32.
    *issued = c->devOpIssued.load();
    const uint32_t entered = c->hostProgress ? *(volatile uint32_t *)c->hostProgress : (uint32_t)*issued;
    *done = *issued - (uint32_t)((uint32_t)*issued - entered);
    if (*done > *issued) *done = *issued;
}

void DumpTaskException(Comm *c, const DevStatus &s)
{
    {
        std::lock_guard<std::mutex> lk(c->dfxMu);
        if (c->exceptionDumped) return;
        c->exceptionDumped = true;
    }
    std::vector<uint8_t> header(kHeapHeaderBytes);
    bool haveHeader = false;
    if (c->backend == BackendKind::SIM) { memcpy(header.data(), c->heap[c->rank], kHeapHeaderBytes); haveHeader = true; }
    else haveHeader = CudaReadHeapHeader(c, header.data(), kHeapHeaderBytes) == HCCL_SUCCESS;
    std::vector<OpRecord> ops;
    {
        std::lock_guard<std::mutex> lk(c->opRingMu);
        size_t n = c->opRing.size(), first = n > 50 ? n - 50 : 0;
        ops.assign(c->opRing.begin() + first, c->opRing.end());
    }
    std::ostringstream rep;
    rep << "task exception on comm " << c->name << " rank " << c->rank << ": code=" << s.code << " peer=" << s.peer << " channel=" << s.channel
        << " phase=" << s.phase << " opSeq=" << s.opSeq << " observed=" << s.observed << " expected=" << s.expected << ". ";
    if (haveHeader) rep << DescribeFlags(s, reinterpret_cast<const DevCtrl *>(header.data()), reinterpret_cast<const DevFlags *>(header.data() + kCtrlBytes), c->nranks);
    else rep << "(the control block could not be copied from the device)";
    rep << ". last " << ops.size() << " operators:";
    for (const OpRecord &r : ops)
        rep << " [" << r.seq << " " << CmdName(r.opType) << " " << r.algName << " count=" << r.count << " " << DataTypeName(r.dtype) << "]";
    const std::string text = rep.str();
    HCCL_ERROR("%s", text.size() > 3500 ? (text.substr(0, 3500) + " ...").c_str() : text.c_str());
    c->counters.exceptionDumps++;
    {
        std::lock_guard<std::mutex> lk(c->dfxMu);
        c->lastExceptionReport = text;
    }
    const char *dir = getenv("HCCL_EXCEPTION_DUMP_DIR");
    if (!dir || !*dir) return;
    BinaryStream bs;
    bs << kDumpMagic << kDumpVersion << c->name << c->rank << c->nranks << s;
    std::vector<uint8_t> hdr = haveHeader ? header : std::vector<uint8_t>();
    bs << hdr;
    std::vector<OpRecordPod> pods;
    for (const OpRecord &r : ops) {
        OpRecordPod p{};
        p.seq = r.seq; p.opType = (uint32_t)r.opType; p.dtype = (uint32_t)r.dtype; p.reduceOp = (uint32_t)r.reduceOp; p.root = r.root; p.engine = r.engine;
        p.count = r.count; memcpy(p.algName, r.algName, sizeof(p.algName)); p.beginNs = r.beginNs; p.endNs = r.endNs;
        pods.push_back(p);
    }
    bs << pods;
    std::string path = std::string(dir) + "/hccl_exception_" + c->name + "_rank" + std::to_string(c->rank) + ".bin";
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) { HCCL_WARNING("cannot write the exception dump %s", path.c_str()); return; }
    f.write(reinterpret_cast<const char *>(bs.Data().data()), (std::streamsize)bs.Data().size());
    HCCL_RUN_INFO("task-exception dump written to %s (%zu bytes)", path.c_str(), bs.Data().size());
}

}  // namespace hccl

using namespace hccl;

extern "C" {

HcclResult HcclGetFaultReports(HcclComm comm, char *stuck, uint32_t stuckLen, char *exception, uint32_t exceptionLen)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(c->dfxMu);
    if (stuck && stuckLen) snprintf(stuck, stuckLen, "%s", c->lastStuckReport.c_str());
    if (exception && exceptionLen) snprintf(exception, exceptionLen, "%s", c->lastExceptionReport.c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclGetFaultCounters(HcclComm comm, uint64_t *opRetries, uint64_t *stuckReports, uint64_t *exceptionDumps)
{
    Comm *c = CommFromHandle(comm);
    if (!c) return HCCL_E_PTR;
    if (opRetries) *opRetries = c->counters.opRetries;
    if (stuckReports) *stuckReports = c->counters.stuckReports;
    if (exceptionDumps) *exceptionDumps = c->counters.exceptionDumps;
    return HCCL_SUCCESS;
}

// Reads a file written by the task-exception dump and renders it as text: the status record, the failing channel's flag
// words, and the recorded operators.
HcclResult HcclReadExceptionDump(const char *path, char *buf, uint32_t bufLen)
{
    if (!path || !buf || bufLen == 0) return HCCL_E_PTR;
    std::ifstream f(path, std::ios::binary);
    if (!f) return HCCL_E_NOT_FOUND;
    std::vector<uint8_t> data((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    try {
        BinaryStream bs(std::move(data));
        uint32_t magic = 0, version = 0, rank = 0, nranks = 0;
        std::string name;
        DevStatus s{};
        std::vector<uint8_t> header;
        bs >> magic >> version;
        if (magic != kDumpMagic || version != kDumpVersion) return HCCL_E_PARA;
        bs >> name >> rank >> nranks >> s >> header;
        std::vector<OpRecordPod> pods;
        bs >> pods;
        std::ostringstream o;
        o << "comm=" << name << " rank=" << rank << "/" << nranks << " code=" << s.code << " peer=" << s.peer << " channel=" << s.channel << " phase=" << s.phase
          << " opSeq=" << s.opSeq << " observed=" << s.observed << " expected=" << s.expected << "\n";
        if (header.size() == kHeapHeaderBytes)
            o << DescribeFlags(s, reinterpret_cast<const DevCtrl *>(header.data()), reinterpret_cast<const DevFlags *>(header.data() + kCtrlBytes), nranks) << "\n";
        o << "operators=" << pods.size() << "\n";
        for (const OpRecordPod &p : pods) o << p.seq << " " << CmdName((HcclCMDType)p.opType) << " " << p.algName << " count=" << p.count << "\n";
        snprintf(buf, bufLen, "%s", o.str().c_str());
    } catch (const std::exception &e) {
        HCCL_ERROR("exception dump %s is damaged: %s", path, e.what());
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

}  // extern "C"
