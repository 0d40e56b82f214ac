// Host helpers shared by the GEMM-based kernels: tensor-map encoding and launch.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "hccl/hccl_types.h"

namespace hccl {
namespace mc2 {

// 2-D row-major tensor [rows, cols] of 2-byte (or 1-byte) elements with row pitch `pitchBytes`; box = boxCols x boxRows,
// 128-byte swizzle (boxCols * elemBytes must be 128).
HcclResult EncodeTmap2D(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t pitchBytes, uint32_t boxRows, uint32_t boxCols,
                        uint32_t elemBytes);
// Scale atoms of a block-scaled operand as a tensor map: [atoms][128 x u32], box = one 512-byte atom, no swizzle.
HcclResult EncodeTmapSf(CUtensorMap *out, const void *scales, uint64_t atoms);
uint32_t *GemmErrorWord();      // device word shared by all GEMM launches of this process (per device)
HcclResult GemmCheckError();    // reads it back (synchronous; tests only)
int SmCount();

}  // namespace mc2
}  // namespace hccl
