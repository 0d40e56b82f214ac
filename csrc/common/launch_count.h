// Process-wide count of kernels this library has launched (GEMM, fused, collective, MoE): benchmarks report the delta over
// their timed region, and a zero delta on a GPU box means a fallback ran instead of the native kernels.
#pragma once
#include <atomic>
#include <stdint.h>

namespace hccl {
inline std::atomic<uint64_t> &KernelLaunchCounter()
{
    static std::atomic<uint64_t> n{0};
    return n;
}
inline void CountLaunch(uint64_t n = 1) { KernelLaunchCounter().fetch_add(n, std::memory_order_relaxed); }
}  // namespace hccl
