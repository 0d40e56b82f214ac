// MXFP8 (OCP microscaling: e4m3 elements, one e8m0 scale per 1 x 32 block) on one GPU: the quantiser that produces the
// operand format of the block-scaled tcgen05 kernels, and the plain GEMM entry on those kernels.
//
// Operand format of a [rows, K] matrix (K a multiple of 128):
//   payload  rows x K bytes, row-major e4m3
//   scales   [ceil(rows / 128)][K / 128][512] bytes: for row r and K block kb (32 elements) the e8m0 scale (a biased power
//            of two, value = 2^(byte - 127)) sits in atom (r / 128, kb / 4) at byte (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4,
//            which is the order tcgen05.cp moves into tensor memory without any shuffle.
// Quantisation rule (OCP MX v1.0): scale = 2^(floor(log2(amax)) - 8) (8 = exponent of the largest e4m3 normal, 448 = 1.75 * 2^8),
// elements = x / scale converted to e4m3 with round-to-nearest-even and saturation; an all-zero block gets scale 2^-127.
// HCCL has no counterpart; its MC2 header only names fp8 data types (reference: include/hccl_mc2.h:31-36, hccl_types.h).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <atomic>
#include "../common/launch_count.h"
#include "../common/log.h"
#include "gemm_host.h"
#include "gemm_sm100_mx.cuh"
#include "gemm_sm100_mx_2cta.cuh"
#include "hccl/hccl_mc2.h"

namespace hccl {
namespace mc2 {

namespace {

// One thread per 1 x 32 block. Threads of a warp take consecutive K blocks of one row, so a warp reads 2 KB of one row.
__global__ void QuantizeMxfp8Kernel(const __nv_bfloat16 *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales, uint32_t rows,
                                    uint32_t rowsPadded, uint32_t K)
{
    const uint32_t kBlocks = K / 32;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)rowsPadded * kBlocks) return;
    const uint32_t r = (uint32_t)(idx / kBlocks), kb = (uint32_t)(idx % kBlocks);
    uint8_t *sf = scales + ((uint64_t)(r / 128) * (K / 128) + kb / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4;
    if (r >= rows) { *sf = 127; return; }                        // padding rows: scale 1, their operands read as zero
    const uint4 *src = (const uint4 *)(in + (uint64_t)r * K + (uint64_t)kb * 32);
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) raw[i] = src[i];
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw[i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(h[j]);
            v[i * 8 + 2 * j] = f.x; v[i * 8 + 2 * j + 1] = f.y;
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    // biased exponent of amax (finite inputs assumed; NaN / Inf saturate through the conversion below)
    int e = (int)((__float_as_uint(amax) >> 23) & 0xff);         // floor(log2(amax)) + 127 for normal amax; 0 for zero / denormal
    int se = e - 8;                                              // scale exponent, biased
    if (se < 0) se = 0;
    if (se > 254) se = 254;
    *sf = (uint8_t)se;
    const float inv = __uint_as_float((uint32_t)(254 - se) << 23);    // 2^(127 - se): exact reciprocal of the scale (se = 0 gives 2^127)
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[i * 4] * inv, v[i * 4 + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[i * 4 + 2] * inv, v[i * 4 + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        packed[i] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    uint4 *dst = (uint4 *)(payload + (uint64_t)r * K + (uint64_t)kb * 32);
    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

template <int BN> HcclResult LaunchPlainMx(const void *a, const void *sfa, const void *b, const void *sfb, void *c, uint32_t M, uint32_t N, uint32_t K, bool outFp32,
                                          cudaStream_t s)
{
    GemmParams p{};
    CHK_RET(EncodeTmap2D(&p.tmapA, a, M, K, (uint64_t)K, kBM, kMxBK, 1));
    CHK_RET(EncodeTmap2D(&p.tmapB, b, N, K, (uint64_t)K, BN, kMxBK, 1));
    p.C = c; p.M = M; p.N = N; p.K = K; p.ldc = N; p.outFp32 = outFp32; p.groupM = 16; p.errorWord = GemmErrorWord();
    p.sfA = (const uint8_t *)sfa; p.sfB = (const uint8_t *)sfb; p.sfAtomsB = (N + 127) / 128; p.elemBytes = 1;
    using S = GemmMxSmem<BN>;
    static std::atomic<bool> attrSet{false};
    auto kern = GemmKernelMx<BN, PlainPolicy, false>;
    size_t smem = S::kTotal + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return HCCL_E_RUNTIME;
        attrSet = true;
    }
    uint32_t tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
    uint32_t grid = std::min<uint32_t>(tiles, (uint32_t)SmCount());
    kern<<<grid, kGemmThreads, smem, s>>>(p, nullptr);
    CountLaunch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("MXFP8 GEMM launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

// CTA pairs (cta_group::2): 256 x BN tiles, one cluster of two CTAs per tile, an even grid.
template <int BN> HcclResult LaunchPlainMxPair(const void *a, const void *sfa, const void *b, const void *sfb, void *c, uint32_t M, uint32_t N, uint32_t K, bool outFp32,
                                              cudaStream_t s)
{
    GemmParams p{};
    using S = GemmMx2CtaSmem<BN>;
    CHK_RET(EncodeTmap2D(&p.tmapA, a, M, K, (uint64_t)K, kBM, kMxBK, 1));
    CHK_RET(EncodeTmap2D(&p.tmapB, b, N, K, (uint64_t)K, BN / 2, kMxBK, 1));
    CHK_RET(EncodeTmapSf(&p.tmapSfA, sfa, (uint64_t)((M + 127) / 128) * (K / 128)));
    CHK_RET(EncodeTmapSf(&p.tmapSfB, sfb, (uint64_t)((N + 127) / 128) * (K / 128)));
    p.C = c; p.M = M; p.N = N; p.K = K; p.ldc = N; p.outFp32 = outFp32; p.groupM = 8; p.errorWord = GemmErrorWord();
    p.sfA = (const uint8_t *)sfa; p.sfB = (const uint8_t *)sfb; p.sfAtomsB = (N + 127) / 128; p.elemBytes = 1;
    static std::atomic<bool> attrSet{false};
    auto kern = GemmKernelMx2Cta<PlainPolicy, BN>;
    size_t smem = S::kTotal + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return HCCL_E_RUNTIME;
        attrSet = true;
    }
    uint32_t tiles = ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + BN - 1) / BN);
    uint32_t pairs = std::min<uint32_t>(tiles, (uint32_t)SmCount() / 2);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pairs * 2);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    CountLaunch();
    if (e != cudaSuccess) { HCCL_ERROR("block-scaled CTA-pair GEMM launch failed: %s", cudaGetErrorString(e)); (void)cudaGetLastError(); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

}  // namespace
}  // namespace mc2
}  // namespace hccl

using namespace hccl;
using namespace hccl::mc2;

extern "C" {

uint64_t HcclMxfp8ScaleBytes(uint64_t rows, uint64_t k) { return ((rows + 127) / 128) * (k / 128) * 512; }

HcclResult HcclQuantizeMxfp8(const void *in, void *payload, void *scales, uint64_t rows, uint64_t k, cudaStream_t stream)
{
    if (!in || !payload || !scales) return HCCL_E_PTR;
    if (rows == 0 || k == 0 || k % 128 || rows > 0x7fffffff || k > 0x7fffffff) {
        HCCL_ERROR("HcclQuantizeMxfp8: K (%llu) must be a non-zero multiple of 128", (unsigned long long)k);
        return HCCL_E_PARA;
    }
    if (((uintptr_t)in & 15u) || ((uintptr_t)payload & 15u)) { HCCL_ERROR("HcclQuantizeMxfp8: buffers must be 16-byte aligned"); return HCCL_E_PARA; }
    const uint64_t rowsPadded = (rows + 127) / 128 * 128;
    const uint64_t threads = rowsPadded * (k / 32);
    QuantizeMxfp8Kernel<<<(uint32_t)((threads + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16 *)in, (uint8_t *)payload, (uint8_t *)scales, (uint32_t)rows,
                                                                             (uint32_t)rowsPadded, (uint32_t)k);
    CountLaunch();
    if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    return HCCL_SUCCESS;
}

// C[M,N] = dequant(A)[M,K] * dequant(B)[N,K]^T; operands in the format above; bf16 or fp32 output. K % 128 == 0, N % 8 == 0.
HcclResult HcclGemmMxfp8(const void *a, const void *sfa, const void *b, const void *sfb, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32,
                         cudaStream_t stream)
{
    if (!a || !sfa || !b || !sfb || !c) return HCCL_E_PTR;
    if (m == 0 || n == 0 || k == 0 || (k % 128) || (n % 8) || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) {
        HCCL_ERROR("HcclGemmMxfp8: unsupported shape %llux%llux%llu (K must be a multiple of 128, N of 8)", (unsigned long long)m, (unsigned long long)n,
                   (unsigned long long)k);
        return HCCL_E_PARA;
    }
    // CTA pairs when the product fills the GPU with pair tiles (HCCL_MX_PAIR=0 keeps the one-CTA kernels): 192-wide tiles with two
    // accumulators, or 256-wide ones when K is long enough to hide their exposed epilogue
    {
        const char *e = getenv("HCCL_MX_PAIR");
        const bool pair = !(e && e[0] == '0') && !getenv("HCCL_MX_TILE_N");
        const uint64_t bn = k >= 16384 ? 256 : 192;
        const uint64_t pairTiles = ((m + 255) / 256) * ((n + bn - 1) / bn);
        if (pair && n >= 256 && pairTiles >= (uint64_t)SmCount() / 2)
            return bn == 256 ? LaunchPlainMxPair<256>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream)
                             : LaunchPlainMxPair<192>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    }
    // HCCL_MX_TILE_N = 192 | 256 picks the wide tile of large products (as for the fused operators)
    if (const char *e = getenv("HCCL_MX_TILE_N")) {
        const int v = atoi(e);
        const uint64_t tiles = ((m + 127) / 128) * ((n + (uint64_t)(v > 0 ? v : 256) - 1) / (uint64_t)(v > 0 ? v : 256));
        if (v == 192 && tiles >= (uint64_t)SmCount()) return LaunchPlainMx<192>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    }
    // 256-wide tiles (one accumulator) when they fill the GPU, 128-wide (two accumulators) otherwise
    uint64_t tiles256 = ((m + 127) / 128) * ((n + 255) / 256);
    if (tiles256 >= (uint64_t)SmCount()) return LaunchPlainMx<256>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    return LaunchPlainMx<128>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
}

HcclResult HcclGemmMxfp8Variant(const void *a, const void *sfa, const void *b, const void *sfb, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32,
                                int tileN, cudaStream_t stream)
{
    if (!a || !sfa || !b || !sfb || !c) return HCCL_E_PTR;
    if (m == 0 || n == 0 || k == 0 || (k % 128) || (n % 8) || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return HCCL_E_PARA;
    if (tileN == 256) return LaunchPlainMx<256>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    // 2256 / 2192: CTA pairs (cta_group::2) with 256- / 192-wide tiles
    if (tileN == 2256) return LaunchPlainMxPair<256>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    if (tileN == 2192) return LaunchPlainMxPair<192>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    if (tileN == 192) return LaunchPlainMx<192>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    if (tileN == 128) return LaunchPlainMx<128>(a, sfa, b, sfb, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    return HcclGemmMxfp8(a, sfa, b, sfb, c, m, n, k, outFp32, stream);
}

}  // extern "C"
