// Communicator: everything the operator layer needs from "below" (HCCL's hcomm contract: identity, CCL buffer,
// peer-addressable memory, keyed engine contexts, threads/streams, channels = flag slots, rank graph, and the
// exchange-info side channel; reference call sites: src/ops/op_common/op_common.cc:951-970,1338,1616,1655).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>
#include "../common/env_config.h"
#include "../topo/topo_info.h"
#include "bootstrap.h"
#include "dev_comm.h"
#include "hccl/hccl_comm.h"

namespace hccl {

enum class BackendKind : uint8_t { SIM = 1, CUDA = 2 };

// Keyed blobs per communicator (HcclEngineCtxCreate/Get/Copy/Destroy in HCCL): caches for topology results,
// resource contexts and launch plans, on the host or in device memory.
struct EngineCtxBlob {
    std::vector<uint8_t> host;
    void *dev = nullptr;
    uint64_t devBytes = 0;
};

// Cross-rank parameter consistency record (reference: alg_param.h:695-706 OpExchangeInfo).
struct OpExchangeInfo {
    uint64_t cclBufferSize;
    uint32_t root;
    uint32_t opType;
    uint32_t engine;
    uint32_t reduceOp;
    uint32_t dataType;
    uint32_t pad;
    uint64_t count;
    uint32_t ctaLimit;
    char group[128];
    char algName[128];
    char tag[128];
};

// Last-op registry entry and counters (DFX).
struct OpRecord {
    uint64_t seq;
    HcclCMDType opType;
    HcclDataType dtype;
    HcclReduceOp reduceOp;
    uint64_t count;
    uint32_t root;
    uint32_t engine;
    char algName[64];
    uint64_t beginNs, endNs;     // host timestamps around the enqueue
    uint32_t devSeq, devLaunches; // first device op-counter value and number of kernels of this operator (CUDA engines)
};

struct CommCounters {
    std::atomic<uint64_t> ops{0}, bytes{0}, timeouts{0}, planCacheHits{0}, planCacheMisses{0}, fallbacks{0},
        consistencyChecks{0}, chunkLoops{0}, kernelsLaunched{0}, opRetries{0}, stuckReports{0}, exceptionDumps{0};
    std::mutex mu;
    std::map<std::string, uint64_t> algoHistogram;
};

struct SymAllocBlock { uint64_t off, bytes; bool used; };

class SimWorker;   // ordered async queue that plays the role of a stream for the host backend

struct Comm {
    uint32_t rank = 0, nranks = 1;
    std::string name;                // group name
    std::thread::id creatorThread;   // disambiguates same-named communicators of one process (ranks as threads)
    uint64_t commId = 0;
    BackendKind backend = BackendKind::SIM;
    int device = -1;
    HcclCommConfig config{};
    AlgEnvConfig env;                // snapshot with per-comm overrides applied
    std::unique_ptr<Bootstrap> boot;
    TopoInfo topo;
    std::atomic<int> status{HCCL_COMM_STATUS_READY};

    // symmetric heap
    uint64_t heapBytes = 0;
    std::vector<char *> heap;        // heap[r] mapped locally; heap[rank] is this rank's own
    char *mcHeap = nullptr;          // NVLS multicast mapping or nullptr
    DevComm devComm{};               // host copy
    DevComm *devCommPtr = nullptr;   // device copy (CUDA) or == &devComm (sim)
    DevStatus *hostStatus = nullptr; // pinned, device-mapped (CUDA) / plain (sim)
    uint32_t *hostProgress = nullptr; // pinned, device-mapped: kernels entered on the device (CUDA only)
    std::atomic<uint64_t> devOpIssued{0};   // kernels issued that advance the device op counter (since create / resume)
    void *backendState = nullptr;    // CudaHeapState* / SimHeapState*
    std::vector<SymAllocBlock> arena;
    std::mutex arenaMu;
    std::map<uint64_t, uint64_t> registered;   // heap offset -> bytes of the windows registered with HcclCommMemReg (under arenaMu)

    // host-engine notify bookkeeping and op parity (sim backend keeps them on the host side of the heap)
    uint64_t opSeq = 0;
    std::unique_ptr<SimWorker> worker;

    // caches
    std::mutex ctxMu;
    std::unordered_map<std::string, EngineCtxBlob> engineCtx;
    std::unordered_map<std::string, int> stickyFallback;      // algTag -> engine that finally worked
    std::unordered_map<std::string, bool> consistencyDone;    // algTag -> checked
    std::shared_ptr<void> fastOps;                            // dispatch core: launch lists of repeated calls (op_common.cc)

    // DFX
    CommCounters counters;
    std::mutex opRingMu;
    std::deque<OpRecord> opRing;     // last 64 ops
    std::thread watchdog;
    std::atomic<bool> watchdogStop{false};
    std::atomic<int> remoteErrorRank{-1}, deadRank{-1};
    std::vector<std::function<void(int)>> stateCallbacks;

    // op retry: the last collective as issued (its buffers stay the caller's), re-run after a wait timeout when every
    // rank stopped at the same operator and its input cannot have been overwritten
    std::mutex retryMu;
    std::shared_ptr<void> retryOp;               // OpParam copy (op_retry.cc)
    uint64_t retrySeq = 0;                       // index of that operator on this communicator
    bool retryInputIntact = false;
    std::atomic<int> injectOpDrop{0};            // tests: the next n operators of this rank are recorded but not run
    std::atomic<bool> inRetry{false};
    // stuck detection / task-exception dump
    std::mutex dfxMu;
    std::string lastStuckReport, lastExceptionReport;
    bool exceptionDumped = false;

    // sub-communicators keep their parent's bootstrap alive
    Comm *parent = nullptr;
    bool destroyed = false;
};

// ---- lifecycle (comm.cc)
// Placement (server, super-pod) that the next CommCreate of this thread gives its rank instead of deriving it from the host: set around
// the creation of a sub-communicator, whose ranks keep the placement they have in the parent, and (host simulation only) around a
// creation from a rank table, whose server list says where each rank sits.
const RankDesc *InheritedPlacement();
void SetInheritedPlacement(const RankDesc *d, bool simOnly = false);     // simOnly: ignored when the communicator runs on GPUs
HcclResult CommCreate(uint32_t nranks, const HcclRootInfo *info, uint32_t rank, const HcclCommConfig *cfg, Comm **out);
HcclResult CommDestroy(Comm *c);
Comm *CommFromHandle(HcclComm h);       // validates the handle (nullptr on garbage)
HcclResult CommCheckReady(Comm *c);     // SUCCESS or HCCL_E_SUSPENDING; also folds in async device errors
HcclResult CommSuspend(Comm *c);
HcclResult CommResume(Comm *c);
HcclResult CommPollAsyncError(Comm *c, HcclResult *asyncErr);

// ---- engine-context store
HcclResult EngineCtxCreate(Comm *c, const std::string &tag, bool onDevice, uint64_t bytes, void **ptr);
HcclResult EngineCtxGet(Comm *c, const std::string &tag, bool onDevice, void **ptr, uint64_t *bytes);
HcclResult EngineCtxCopy(Comm *c, const std::string &tag, const void *src, uint64_t bytes);  // host -> device blob
HcclResult EngineCtxDestroy(Comm *c, const std::string &tag);

// ---- symmetric arena
HcclResult SymAlloc(Comm *c, uint64_t bytes, void **ptr);
HcclResult SymFree(Comm *c, void *ptr);
bool SymContains(Comm *c, const void *ptr, uint64_t bytes);
uint64_t SymOffsetOf(Comm *c, const void *ptr);
// Registered windows (HcclCommMemReg): ranges of the symmetric heap the zero-copy kernels may address on every rank.
void AllocatorCommDetach(Comm *c);   // res_api.cc: forget `c` as the communicator behind HcclAllocHook / HcclFreeHook
HcclResult CommRegisterWindow(Comm *c, const void *ptr, uint64_t bytes, uint64_t *off);
HcclResult CommDeregisterWindow(Comm *c, const void *ptr);
bool CommRegisteredOffset(Comm *c, const void *ptr, uint64_t bytes, uint64_t *off);

// ---- backend hooks (backend_sim.cc / backend_cuda.cc)
HcclResult SimBackendInit(Comm *c);
void SimBackendDestroy(Comm *c);
HcclResult CudaBackendInit(Comm *c);
void CudaBackendDestroy(Comm *c);
HcclResult CudaBackendResetFlags(Comm *c);
HcclResult CudaBackendQuiesce(Comm *c);
bool CudaDeviceAvailable(int *currentDevice);

// ---- fault handling (dfx/fault_handling.cc, exec/op_retry.cc)
bool OpRetryEnabled(const Comm *c);
HcclResult CommOpRetry(Comm *c);                       // collective: agree, resume, re-issue; HCCL_E_OPRETRY_FAIL when it cannot
void DumpTaskException(Comm *c, const DevStatus &s);   // flag arena + last operators -> log (and HCCL_EXCEPTION_DUMP_DIR)
void CommProgress(Comm *c, uint64_t *issued, uint64_t *done);
HcclResult CudaReadHeapHeader(Comm *c, void *hostDst, uint64_t bytes);   // device -> host copy on a private stream
// ---- DFX
std::string LifecycleLogTake();   // and clears it
void RecordOp(Comm *c, const OpRecord &r);
void StartWatchdog(Comm *c);
void StopWatchdog(Comm *c);

// Sim stream: ordered async execution
class SimWorker {
public:
    SimWorker();
    ~SimWorker();
    void Enqueue(std::function<HcclResult()> fn);
    HcclResult Drain();                 // waits; returns the first error since the previous Drain
    uint64_t Enqueued() const { return enqueued_.load(); }
    uint64_t Completed() const { return completed_.load(); }
private:
    void Run();
    std::thread th_;
    std::mutex mu_;
    std::condition_variable cv_, idleCv_;
    std::deque<std::function<HcclResult()>> q_;
    bool stop_ = false, busy_ = false;
    std::atomic<uint64_t> enqueued_{0}, completed_{0};
    HcclResult firstErr_ = HCCL_SUCCESS;
};

}  // namespace hccl
