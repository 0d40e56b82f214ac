#include "slice_planner.h"
#include <algorithm>
#include <cmath>

namespace hccl {
namespace {

// Bytes one rank sends on each level, per byte of the planned quantity, for a share that starts on level 0 (f0) and for
// one that starts on level 1 (f1). X, Y = group sizes of level 0 and 1.
struct Coeff { double l0f0, l0f1, l1f0, l1f1; uint32_t calls0f0, calls1f0, calls0f1, calls1f1; };

Coeff CoeffFor(PipeOp op, double X, double Y)
{
    Coeff c{};
    switch (op) {
        case PipeOp::ALLGATHER:
            // f0: gather my block inside the server, then forward the server's X blocks between servers
            // f1: gather my block between servers, then forward the Y blocks inside the server
            c.l0f0 = X - 1; c.l1f0 = X * (Y - 1);
            c.l1f1 = Y - 1; c.l0f1 = Y * (X - 1);
            c.calls0f0 = 1; c.calls1f0 = (uint32_t)X; c.calls1f1 = 1; c.calls0f1 = (uint32_t)Y;
            break;
        case PipeOp::REDUCE_SCATTER:
            // the mirror image: the first stage works on the other level's whole set of blocks
            c.l0f0 = Y * (X - 1); c.l1f0 = Y - 1;
            c.l1f1 = X * (Y - 1); c.l0f1 = X - 1;
            c.calls0f0 = (uint32_t)Y; c.calls1f0 = 1; c.calls1f1 = (uint32_t)X; c.calls0f1 = 1;
            break;
        case PipeOp::ALLREDUCE:
            // reduce-scatter on the first level, all-reduce of the slice on the second, all-gather on the first
            c.l0f0 = 2 * (X - 1) / X; c.l1f0 = 2 * (Y - 1) / (X * Y);
            c.l1f1 = 2 * (Y - 1) / Y; c.l0f1 = 2 * (X - 1) / (X * Y);
            c.calls0f0 = 2; c.calls1f0 = 1; c.calls1f1 = 2; c.calls0f1 = 1;
            break;
    }
    return c;
}

uint64_t AlignDown(uint64_t v, uint64_t a) { return v / a * a; }

}  // namespace

void StepRange(const PipeShare &s, uint64_t align, uint32_t i, uint64_t *off, uint64_t *bytes)
{
    const uint64_t per = std::max<uint64_t>(align, AlignDown(s.bytes / std::max(1u, s.steps), align));
    const uint64_t lo = std::min<uint64_t>(s.bytes, per * i);
    const uint64_t hi = i + 1 == s.steps ? s.bytes : std::min<uint64_t>(s.bytes, per * (i + 1));
    *off = s.off + lo;
    *bytes = hi - lo;
}

HcclResult PlanSlices(PipeOp op, const AxisSpec &level0, const AxisSpec &level1, uint64_t bytesPerRank, uint64_t align, uint32_t maxSteps, SlicePlan *out)
{
    if (!out || align == 0 || level0.ranks == 0 || level1.ranks == 0 || level0.bandwidthGBs <= 0 || level1.bandwidthGBs <= 0) return HCCL_E_PARA;
    *out = SlicePlan{};
    const double X = level0.ranks, Y = level1.ranks, S = (double)bytesPerRank;
    const double us0 = 1e-3 / level0.bandwidthGBs, us1 = 1e-3 / level1.bandwidthGBs;        // microseconds per byte
    const Coeff c = CoeffFor(op, X, Y);
    // the Sequence executor's order: all-gather starts between the servers, the reductions start inside the server
    const bool seqStartsOn1 = op == PipeOp::ALLGATHER;
    const double seqLoad0 = S * (seqStartsOn1 ? c.l0f1 : c.l0f0) * us0, seqLoad1 = S * (seqStartsOn1 ? c.l1f1 : c.l1f0) * us1;
    const double seqLat = seqStartsOn1 ? c.calls1f1 * level1.latencyUs + c.calls0f1 * level0.latencyUs : c.calls0f0 * level0.latencyUs + c.calls1f0 * level1.latencyUs;
    out->sequenceUs = seqLoad0 + seqLoad1 + seqLat;
    if (level0.ranks == 1 || level1.ranks == 1 || bytesPerRank < 2 * align) {
        out->shares.assign(1, PipeShare{0, bytesPerRank, seqStartsOn1 ? 1u : 0u, 1});
        out->parallelUs = out->sequenceUs;
        out->loadUs[0] = seqLoad0; out->loadUs[1] = seqLoad1;
        return HCCL_SUCCESS;
    }

    // a = fraction of the block in the share that starts on level 0. Loads are linear in a; the larger of the two is
    // smallest where they cross (or at an end of [0, 1] when they do not cross inside it: then one share takes everything
    // and only its steps overlap the two levels).
    auto load0 = [&](double a) { return S * (a * c.l0f0 + (1 - a) * c.l0f1) * us0; };
    auto load1 = [&](double a) { return S * (a * c.l1f0 + (1 - a) * c.l1f1) * us1; };
    const double slope = (c.l0f0 - c.l0f1) * us0 - (c.l1f0 - c.l1f1) * us1;
    double best = 0;
    if (std::fabs(slope) > 1e-30) best = std::min(1.0, std::max(0.0, (c.l1f1 * us1 - c.l0f1 * us0) / slope));
    for (double a : {0.0, 1.0})
        if (std::max(load0(a), load1(a)) < std::max(load0(best), load1(best))) best = a;
    uint64_t bytes0 = AlignDown((uint64_t)std::llround(best * S), align);
    if (bytes0 > bytesPerRank) bytes0 = AlignDown(bytesPerRank, align);
    const uint64_t bytes1 = bytesPerRank - bytes0;

    const uint64_t minStep = std::max<uint64_t>(align, 64u << 10);
    auto stepsFor = [&](uint64_t b) { return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(std::max(1u, maxSteps), b / minStep)); };
    uint32_t steps0 = 0, steps1 = 0;
    if (bytes0) { steps0 = stepsFor(bytes0); out->shares.push_back(PipeShare{0, bytes0, 0, steps0}); }
    if (bytes1) { steps1 = stepsFor(bytes1); out->shares.push_back(PipeShare{bytes0, bytes1, 1, steps1}); }
    const double a = (double)bytes0 / S;
    // every template call is one synchronised step of its level; calls of one level run one after the other
    const double lat0 = (steps0 * c.calls0f0 + steps1 * c.calls0f1) * level0.latencyUs;
    const double lat1 = (steps0 * c.calls1f0 + steps1 * c.calls1f1) * level1.latencyUs;
    out->loadUs[0] = load0(a) + lat0;
    out->loadUs[1] = load1(a) + lat1;
    // what cannot overlap: one step of the less loaded level at the ends of the pipeline
    const double edge = std::min(out->loadUs[0], out->loadUs[1]) / std::max(steps0, steps1);
    out->parallelUs = std::max(out->loadUs[0], out->loadUs[1]) + edge;
    return HCCL_SUCCESS;
}

}  // namespace hccl
