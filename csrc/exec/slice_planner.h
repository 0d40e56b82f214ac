// Slice planner for operators that run on two levels of the topology at once.
//
// A two-level operator that finishes one level before it starts the next (the Sequence executor) leaves one level's
// links idle at any time. The Parallel executor cuts every rank's block into two shares that cross the levels in opposite
// orders, so both levels carry traffic from the first step to the last, and cuts each share into steps so that the second
// stage of a step overlaps the first stage of the next. This planner decides the cut: it balances the bytes the two shares
// put on each level against that level's bandwidth, aligns the cut, picks the step count, and prices both forms so that the
// selector can compare them.
//
// HCCL's counterpart is the OmniPipe slice calculation (reference: src/ops/op_common/omnipipe_data_slice_calc.h:27-42
// for its per-link bandwidth constants, :75-110 for the inputs it takes, omnipipe_data_slice_calc.cc:145-223 for the
// per-step sizes of its 2-D all-gather). Its step sizes follow a geometric series in the bandwidth ratio; here the two
// shares are balanced in closed form and the steps of a share are equal, which is enough when every level is a full mesh
// (NVSwitch inside a server, a rail-optimised fabric between servers).
#pragma once
#include <cstdint>
#include <vector>
#include "hccl/hccl_types.h"

namespace hccl {

enum class PipeOp : uint8_t { ALLGATHER = 0, REDUCE_SCATTER = 1, ALLREDUCE = 2 };

struct AxisSpec {
    uint32_t ranks = 1;          // group size on this level
    double bandwidthGBs = 1.0;   // per rank and direction on this level
    double latencyUs = 2.0;      // one synchronised step on this level
};

struct PipeShare {
    uint64_t off = 0, bytes = 0; // byte range of every rank's block this share carries
    uint32_t firstLevel = 0;     // the level its first stage runs on (the second stage runs on the other one)
    uint32_t steps = 1;          // equal steps the share is cut into (the last one takes the remainder)
};

struct SlicePlan {
    std::vector<PipeShare> shares;           // shares with bytes == 0 are left out; one share = nothing to balance
    double sequenceUs = 0, parallelUs = 0;   // modelled completion times of the two forms
    double loadUs[2] = {0, 0};               // time each level is busy in the parallel form
};

// bytesPerRank: AllGather / ReduceScatter: one rank's block; AllReduce: the whole vector. align: share and step boundaries are
// multiples of it (a multiple of the element size). maxSteps bounds the steps per share (HCCL uses at most 5).
HcclResult PlanSlices(PipeOp op, const AxisSpec &level0, const AxisSpec &level1, uint64_t bytesPerRank, uint64_t align, uint32_t maxSteps, SlicePlan *out);

// Byte range of step `i` of a share.
void StepRange(const PipeShare &s, uint64_t align, uint32_t i, uint64_t *off, uint64_t *bytes);

}  // namespace hccl
