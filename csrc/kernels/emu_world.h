// Single-GPU emulation world shared by the collective and fused-kernel test entry points: every rank's heap lives on
// the current device and one cooperative launch (blockIdx.y = rank) covers all ranks.
#pragma once
#include <vector>
#include "../core/dev_comm.h"
#include "coll_args.h"

namespace hccl {

struct EmuWorld {
    int nranks = 0;
    std::vector<char *> heaps;
    DevComm *devComms = nullptr;
    std::vector<DevComm> hostComms;
    DevStatus *status = nullptr;       // pinned, one per rank
    CollArgs *devArgs = nullptr;
    BatchArgs *devBatch = nullptr;
    void *devFusedParams = nullptr;    // GemmParams[nranks] for the fused kernels
    uint64_t cclBytes = 0, mailboxBytes = 0, arenaOff = 0, arenaBytes = 0;
};

}  // namespace hccl
