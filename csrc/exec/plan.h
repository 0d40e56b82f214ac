// Schedule IR: what an algorithm template emits and what the host engines, the copy-engine executor and the
// offline checker consume.
//
// The vocabulary is the one HCCL's host/AICPU templates speak through their data-transfer wrapper and that its
// offline "algorithm analyzer" records as task stubs (reference: src/ops/op_common/template/wrapper/
// alg_data_trans_wrapper.cc:127-154,249-300,815-834; test/st/algorithm/utils/src/sim_world/sim_task.h:22-23):
// one-sided WRITE / READ with optional inline reduce, local copy / reduce, and counting notifies between ranks
// (POST / WAIT) and between the queues of one rank (LOCAL_POST / LOCAL_WAIT).
#pragma once
#include <cstdint>
#include <string>
#include <vector>
#include "hccl/hccl_types.h"

namespace hccl {

// CCL = this op's scratch half in the heap; MAILBOX = the point-to-point staging area (offset relative to its base)
// ABS = `off` holds an absolute local address (BatchSendRecv items each bring their own buffer)
enum class BufKind : uint8_t { INPUT = 0, OUTPUT = 1, CCL = 2, MAILBOX = 3, ABS = 4 };

struct BufRef {
    BufKind kind = BufKind::CCL;
    uint64_t off = 0;            // bytes from the start of the buffer
};

enum class TaskType : uint8_t {
    LOCAL_COPY, LOCAL_REDUCE,    // dst (local) <- src (local)          / dst = dst (op) src
    WRITE, WRITE_REDUCE,         // remote CCL <- local src              / remote = remote (op) src
    READ, READ_REDUCE,           // local dst <- remote CCL              / dst = dst (op) remote
    POST, WAIT,                  // notify peer `rank` on `slot`         / wait for the next notify from peer
    LOCAL_POST, LOCAL_WAIT       // notify queue `rank` (same rank)      / wait for the next notify from that queue
};

struct Task {
    TaskType type;
    uint32_t rank = 0;           // remote rank (or queue id for LOCAL_*)
    uint32_t slot = 0;           // notify slot
    BufRef dst, src;             // for WRITE the dst is in the remote CCL, for READ the src is
    uint64_t bytes = 0;
};

// One rank's schedule for one chunk: queue 0 is the "main thread" bound to the caller's stream, further
// queues are helper threads that run concurrently (HCCL's slave threads).
struct Plan {
    std::vector<std::vector<Task>> queues;
    HcclDataType dtype = HCCL_DATA_TYPE_FP32;
    HcclReduceOp op = HCCL_REDUCE_SUM;
    void EnsureQueues(size_t n) { if (queues.size() < n) queues.resize(n); }
    size_t TaskCount() const { size_t n = 0; for (auto &q : queues) n += q.size(); return n; }
};

const char *TaskTypeName(TaskType t);
std::string DumpPlan(const Plan &p, uint32_t rank);

}  // namespace hccl
