// TCP bootstrap: rendezvous, small collectives (allgather / barrier / broadcast), a key-value store and a
// heartbeat channel, all through a service thread that lives in the process of rank 0.
//
// HCCL's control plane (root listens on a host socket, ranks connect, exchange device info, heartbeat links;
// reference: docs/zh/user_guide/fault_diagnosis/task_exec_stage.md:18-28 and the HcclGetRootInfo /
// HcclCommInitRootInfo usage in examples/02_collectives/01_allreduce/main.cc:77,122) is re-done as a star around a
// poll()-driven service: 8 ranks on one box never stress it, and one code path serves thread-per-GPU and
// process-per-GPU callers alike. File descriptors of CUDA VMM allocations travel separately over abstract unix
// sockets (SendFds / RecvFds) because TCP cannot carry SCM_RIGHTS.
#pragma once
#include <atomic>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include "hccl/hccl_types.h"

namespace hccl {

struct RootInfoBlob {           // lives inside HcclRootInfo::internal
    uint32_t magic;             // 'HCB2'
    uint32_t port;
    uint64_t nonce;
    int32_t pid;
    char ip[64];
};
constexpr uint32_t kRootMagic = 0x32424348u;

struct HeartbeatMsg {
    int32_t error;         // 0 = fine; a device / host-engine status code otherwise
    uint32_t clearError;   // 1 = forget the recorded root-cause error (sent by rank 0 while the group resumes)
    uint64_t opsIssued;    // operators this rank has issued on the communicator
    uint64_t opsDone;      // operators this rank knows to have completed
};
struct HeartbeatReply {
    int32_t deadRank;      // -1 none; rank whose heartbeat is older than the LOST threshold
    int32_t errorRank;     // -1 none; first rank that reported an error (root cause broadcast)
    int32_t errorCode;
    uint32_t aliveMask;    // bit r set when rank r has an open heartbeat connection
    int32_t lagRank;       // rank that has completed the fewest operators (-1 before every rank has reported)
    uint32_t pad;
    uint64_t lagDone;      // ... and how many it has completed
    uint64_t maxIssued;    // most operators any rank has issued
};

class BootstrapRoot;  // service side

class Bootstrap {
public:
    Bootstrap() = default;
    ~Bootstrap();
    // Creates the listener for a future root (rank 0) and fills the blob.
    static HcclResult CreateRootInfo(HcclRootInfo *out);
    // Connects to the root named by `info`; rank 0 also starts the service thread on the registered listener.
    HcclResult Init(const HcclRootInfo &info, uint32_t rank, uint32_t nranks, uint32_t timeoutSec, bool heartbeat);
    HcclResult AllGather(const void *in, size_t bytesEach, void *out);
    HcclResult Barrier();
    HcclResult Broadcast(void *buf, size_t bytes, uint32_t root);
    HcclResult Put(const std::string &key, const void *val, size_t bytes);
    HcclResult Get(const std::string &key, std::vector<uint8_t> *val, uint32_t timeoutSec);
    // Heartbeat (second connection): report liveness and an optional error; learn about dead / failed peers.
    HcclResult Heartbeat(const HeartbeatMsg &msg, HeartbeatReply *reply);
    HcclResult Heartbeat(int32_t myError, HeartbeatReply *reply) { HeartbeatMsg m{myError, 0, 0, 0}; return Heartbeat(m, reply); }
    uint32_t Rank() const { return rank_; }
    uint32_t Size() const { return nranks_; }
    uint64_t Nonce() const { return nonce_; }
    void Close();
    // fault injection for tests: drop the next n outgoing allgather contributions of this rank
    void InjectDropNext(int n) { dropNext_ = n; }

private:
    HcclResult Request(int fd, uint32_t op, uint64_t seq, const void *payload, size_t len, std::vector<uint8_t> *reply,
                       uint32_t timeoutSec);
    int fd_ = -1, hbFd_ = -1;
    uint32_t rank_ = 0, nranks_ = 1, timeoutSec_ = 120;
    uint64_t nonce_ = 0, seq_ = 0;
    std::mutex mu_, hbMu_;
    std::shared_ptr<BootstrapRoot> root_;
    std::atomic<int> dropNext_{0};
};

// Unix-socket file-descriptor exchange between ranks on one host. Every rank listens on the abstract address
// "hcclb200-<nonce>-<tag>-<rank>" and serves its descriptor list to every peer that connects.
class FdExchange {
public:
    // Serves `fds` to (nranks-1) peers in a helper thread, and collects each peer's descriptors.
    // out[r] holds rank r's descriptors (own rank: copies of the local fds, not dup'ed).
    static HcclResult AllGatherFds(uint64_t nonce, const std::string &tag, uint32_t rank, uint32_t nranks,
                                   const std::vector<int> &fds, std::vector<std::vector<int>> *out, Bootstrap *boot,
                                   uint32_t timeoutSec);
};

}  // namespace hccl
