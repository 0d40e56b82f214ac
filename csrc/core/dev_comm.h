// Device-visible communicator description and the layout of the symmetric heap.
//
// Every rank owns one heap of identical layout; rank r's heap is mapped into every peer's address space
// (heap[r]) and, when the NVSwitch multicast object could be created, all heaps are also reachable through one
// multicast address (mcHeap) for multimem.* instructions. This is the B200 form of what HCCL's vector-core
// kernels get from the host as GM_IN/GM_OUT peer tables plus a flag area (reference:
// src/ops/op_common/template/aiv/aiv_communication_base_v2.h:158-162,271-291; host side
// src/ops/op_common/op_common.cc:1945-1998).
//
// Synchronisation state lives on the device so that a captured CUDA graph replays correctly: each CTA channel
// keeps its own epoch in the control block, flags only ever grow, and the ping-pong parity of the CCL scratch
// is derived from a device-resident op counter that the last CTA of every collective kernel advances.
#pragma once
#include <stdint.h>

namespace hccl {

constexpr int kMaxRanks = 32;
constexpr int kMaxChannels = 256;       // CTA channels with independent flag rows / epochs
constexpr int kPipeChannels = 128;      // channels of the pipelined (warp-specialised) collectives
constexpr int kNotifySlots = 24;        // host-engine notify counters per peer
constexpr int kP2pCtas = 8;             // CTAs per point-to-point transfer
constexpr uint64_t kCtrlBytes = 64 << 10;
constexpr uint64_t kFlagBytes = (1 << 20) - kCtrlBytes;
constexpr uint64_t kHeapHeaderBytes = 1 << 20;

// Status word written by a kernel that gave up waiting (pinned host memory, device-mapped).
struct DevStatus {
    uint32_t code;      // 0 ok, 1 wait timeout, 2 bounds check, 3 argument error
    uint32_t rank;
    uint32_t peer;
    uint32_t channel;
    uint32_t phase;
    uint32_t opSeq;
    uint32_t observed;  // flag value seen when giving up
    uint32_t expected;
};

// Device-side trace: one record per collective / fused kernel, written by CTA 0 of the kernel from %globaltimer.
constexpr int kTraceSlots = 512;
struct DevTraceRec {
    uint32_t seq;            // op counter value the kernel ran as (kernels since the communicator was created or resumed)
    uint32_t barriers;       // sync points CTA 0 has passed
    uint64_t tEnter;         // ns: CTA 0 entered the kernel
    uint64_t tBarrier[2];    // ns: CTA 0 left its first / last all-rank synchronisation
    uint64_t tLeave;         // ns: CTA 0 left the kernel (0 while it runs, or if it gave up)
};

// Control block at heap offset 0.
struct DevCtrl {
    uint32_t opCount;                 // collectives completed on this rank (parity selects the CCL half)
    uint32_t ticket;                  // CTAs that have read opCount in the running kernel
    uint32_t abortFlag;               // set by the first CTA that timed out; others leave early
    uint32_t gridBar[2];              // software grid barrier (count, generation) for persistent kernels
    uint32_t pad0[3];
    uint32_t chanEpoch[kMaxChannels]; // per-channel barrier epoch
    uint64_t p2pSendSeq[kMaxRanks][kP2pCtas];   // mailbox rounds sent to peer r by p2p CTA b
    uint64_t p2pRecvSeq[kMaxRanks][kP2pCtas];   // mailbox rounds received from peer r by p2p CTA b
    uint64_t hostNotifySent[kMaxRanks][kNotifySlots];   // host-engine: posts issued towards peer r
    uint64_t hostNotifyWaited[kMaxRanks][kNotifySlots]; // host-engine: waits consumed from peer r
    uint32_t pipeEpoch[kPipeChannels];                  // pipelined collectives: flag value reached by the previous operator
    DevTraceRec trace[kTraceSlots];                     // ring indexed by seq % kTraceSlots
};
static_assert(sizeof(DevCtrl) <= kCtrlBytes, "control block too large");

// Flag arena (heap offset kCtrlBytes). Written by peers, read locally.
struct DevFlags {
    uint32_t barrier[kMaxChannels][kMaxRanks];   // barrier[ch][src] = epoch reached by src on channel ch
    uint32_t chunk[kMaxChannels][kMaxRanks];     // chunk[ch][src] = chunks delivered by src on channel ch
    uint64_t p2pData[kMaxRanks][kP2pCtas * 2];   // [src][cta*2+slot] = round number whose data is staged at src
    uint64_t p2pAck[kMaxRanks][kP2pCtas * 2];    // [dst][cta*2+slot] = round number dst has consumed
    uint64_t hostNotify[kMaxRanks][kNotifySlots];// host-engine notify counters, [src][slot]
    // fused-kernel counters, one set per op parity; the owner zeroes its set when the op ends
    uint32_t mc2Ready[2][kMaxRanks][64];         // [half][src][block]: pieces of `block` delivered by src
    uint32_t mc2Done[2][kMaxRanks][4];           // [half][src][k]: second-stage counters (results delivered by src)
    uint32_t moeCount[kMaxRanks][320];           // MoE dispatch: moeCount[src][e] = tokens rank src routes to expert e
    uint32_t pipe[3][kPipeChannels][kMaxRanks];  // pipelined collectives: [staged|moved|drained][ch][src] = sub-chunks done by src
};
static_assert(sizeof(DevFlags) <= kFlagBytes, "flag arena too large");

struct DevComm {
    int32_t rank;
    int32_t nranks;
    uint64_t heapBytes;
    char *heap[kMaxRanks];      // heap[r]: rank r's heap as mapped here (heap[rank] is local)
    char *mcHeap;               // multicast mapping of all heaps, or nullptr
    uint64_t cclOff[2];         // two CCL scratch halves (ping-pong by op parity)
    uint64_t cclBytes;          // bytes per half
    uint64_t mailboxOff;        // p2p staging: [peer][slot] regions of mailboxBytes each
    uint64_t mailboxBytes;
    uint64_t arenaOff;          // user / workspace arena (HcclCommSymAlloc)
    uint64_t arenaBytes;
    uint64_t timeoutNs;         // bound of every device-side wait
    DevStatus *status;          // device-mapped pinned host memory
    int32_t emuRanks;           // > 0: all ranks live on this GPU and one launch covers them (tests)
    int32_t traceOn;            // != 0: CTA 0 of every kernel stamps DevCtrl::trace
    uint32_t *progress;         // device-mapped pinned host word: kernels entered so far (read by the host watchdog); may be null
};

#if defined(__CUDACC__) || defined(HCCL_DEV_HELPERS)
__host__ __device__ inline DevCtrl *CtrlOf(char *heapBase) { return reinterpret_cast<DevCtrl *>(heapBase); }
__host__ __device__ inline DevFlags *FlagsOf(char *heapBase) { return reinterpret_cast<DevFlags *>(heapBase + kCtrlBytes); }
#else
inline DevCtrl *CtrlOf(char *heapBase) { return reinterpret_cast<DevCtrl *>(heapBase); }
inline DevFlags *FlagsOf(char *heapBase) { return reinterpret_cast<DevFlags *>(heapBase + kCtrlBytes); }
#endif

}  // namespace hccl
