// Plain bf16 GEMM entry (C = A * B^T, both K-major) on the tcgen05 kernel, and the helpers the fused ops share.
#include "../common/launch_count.h"
#include <atomic>
#include <mutex>
#include "../common/log.h"
#include "gemm_host.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100_2cta.cuh"
#include <cstdlib>
#include "hccl/hccl_mc2.h"

namespace hccl {
namespace mc2 {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn GetEncode()
{
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        cudaDriverEntryPointQueryResult q;
        void *p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeFn)p;
        else (void)cudaGetLastError();
    });
    return fn;
}
}  // namespace

HcclResult EncodeTmap2D(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t pitchBytes, uint32_t boxRows, uint32_t boxCols,
                        uint32_t elemBytes)
{
    EncodeFn enc = GetEncode();
    if (!enc) { HCCL_ERROR("cuTensorMapEncodeTiled is unavailable"); return HCCL_E_UNAVAIL; }
    if (((uintptr_t)base & 15u) || (pitchBytes & 15u) || boxCols * elemBytes != 128 || boxRows > 256) {
        HCCL_ERROR("tensor map: base %p / pitch %llu must be 16-byte aligned, box %ux%u", base, (unsigned long long)pitchBytes, boxRows, boxCols);
        return HCCL_E_PARA;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitchBytes};
    cuuint32_t box[2] = {boxCols, boxRows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = elemBytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUresult r = enc(out, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { HCCL_ERROR("cuTensorMapEncodeTiled failed: %d", (int)r); return HCCL_E_DRV; }
    return HCCL_SUCCESS;
}

HcclResult EncodeTmapSf(CUtensorMap *out, const void *scales, uint64_t atoms)
{
    EncodeFn enc = GetEncode();
    if (!enc) { HCCL_ERROR("cuTensorMapEncodeTiled is unavailable"); return HCCL_E_UNAVAIL; }
    if (((uintptr_t)scales & 15u) || atoms == 0) { HCCL_ERROR("scale-atom tensor map: base %p must be 16-byte aligned", scales); return HCCL_E_PARA; }
    cuuint64_t dims[2] = {128, atoms};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, 1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(scales), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { HCCL_ERROR("cuTensorMapEncodeTiled (scale atoms) failed: %d", (int)r); return HCCL_E_DRV; }
    return HCCL_SUCCESS;
}

uint32_t *GemmErrorWord()
{
    static uint32_t *w[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!w[dev]) {
        cudaMalloc((void **)&w[dev], 4);
        cudaMemset(w[dev], 0, 4);
    }
    return w[dev];
}

HcclResult GemmCheckError()
{
    uint32_t v = 0;
    if (cudaMemcpy(&v, GemmErrorWord(), 4, cudaMemcpyDeviceToHost) != cudaSuccess) return HCCL_E_RUNTIME;
    if (v) { cudaMemset(GemmErrorWord(), 0, 4); return HCCL_E_TIMEOUT; }
    return HCCL_SUCCESS;
}

// HCCL_GEMM_GROUP_M overrides the rasterisation group (row blocks, or row-block pairs for the CTA-pair kernel) for tuning runs.
static uint32_t GroupMOverride(uint32_t dflt)
{
    static const int v = [] { const char *e = getenv("HCCL_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();
    return v > 0 ? (uint32_t)v : dflt;
}

// HCCL_GEMM_WAIT_SLEEP_NS: nanoseconds the producer / epilogue waits sleep between polls. Default 0 = spin: on the
// 8192 x 28672 x 8192 step a 200 ns back-off measured 1.6 % slower and 1000 ns 6 % slower (the wake-up latency lands on the
// critical path at every tile boundary), so sleeping saves no clock under the power cap.
uint32_t GemmWaitSleepNs()
{
    static const int v = [] { const char *e = getenv("HCCL_GEMM_WAIT_SLEEP_NS"); return e ? atoi(e) : 0; }();
    return (uint32_t)(v > 0 ? v : 0);
}

// HCCL_GEMM_WAIT_HINT_NS / HCCL_GEMM_EPI_SLEEP_NS: suspend-time hint of the CTA-pair kernel's barrier waits and the back-off
// of its epilogue warps while the next accumulator is being computed.
uint32_t GemmWaitHintNs()
{
    static const int v = [] { const char *e = getenv("HCCL_GEMM_WAIT_HINT_NS"); return e ? atoi(e) : 0; }();
    return (uint32_t)(v > 0 ? v : 0);
}
uint32_t GemmEpiSleepNs()
{
    static const int v = [] { const char *e = getenv("HCCL_GEMM_EPI_SLEEP_NS"); return e ? atoi(e) : 0; }();
    return (uint32_t)(v > 0 ? v : 0);
}

int SmCount()
{
    static int n[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    return n[dev];
}

template <int BN> static HcclResult LaunchPlain(const void *a, const void *b, void *c, uint32_t M, uint32_t N, uint32_t K, bool outFp32, cudaStream_t s)
{
    GemmParams p{};
    CHK_RET(EncodeTmap2D(&p.tmapA, a, M, K, (uint64_t)K * 2, kBM, kBK, 2));
    CHK_RET(EncodeTmap2D(&p.tmapB, b, N, K, (uint64_t)K * 2, BN, kBK, 2));
    p.C = c; p.M = M; p.N = N; p.K = K; p.ldc = N; p.outFp32 = outFp32; p.groupM = GroupMOverride(16); p.errorWord = GemmErrorWord(); p.waitSleepNs = GemmWaitSleepNs();
    using S = GemmSmem<BN>;
    static std::atomic<bool> attrSet{false};
    auto kern = GemmKernel<BN, PlainPolicy, false>;
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
    if (e != cudaSuccess) { HCCL_ERROR("GEMM launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

// 256 x 256 tiles on CTA pairs (cta_group::2). Needs an even grid; one cluster of two CTAs per tile.
template <int BN> static HcclResult LaunchPlain2CtaT(const void *a, const void *b, void *c, uint32_t M, uint32_t N, uint32_t K, bool outFp32, cudaStream_t s)
{
    GemmParams p{};
    using S = Gemm2CtaSmemT<BN>;
    CHK_RET(EncodeTmap2D(&p.tmapA, a, M, K, (uint64_t)K * 2, kBM, kBK, 2));
    CHK_RET(EncodeTmap2D(&p.tmapB, b, N, K, (uint64_t)K * 2, S::BN / 2, kBK, 2));
    p.C = c; p.M = M; p.N = N; p.K = K; p.ldc = N; p.outFp32 = outFp32; p.groupM = GroupMOverride(8); p.errorWord = GemmErrorWord(); p.waitHintNs = GemmWaitHintNs(); p.epiSleepNs = GemmEpiSleepNs();
    static std::atomic<bool> attrSet{false};
    auto kern = GemmKernel2Cta<PlainPolicy, BN>;
    size_t smem = S::kTotal + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return HCCL_E_RUNTIME;
        attrSet = true;
    }
    uint32_t tiles = ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + S::BN - 1) / S::BN);
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
    if (e != cudaSuccess) { HCCL_ERROR("2-CTA GEMM launch failed: %s", cudaGetErrorString(e)); (void)cudaGetLastError(); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

static HcclResult LaunchPlain2Cta(const void *a, const void *b, void *c, uint32_t M, uint32_t N, uint32_t K, bool outFp32, cudaStream_t s)
{
    // 224-wide tiles when they waste fewer waves (e.g. N = 3584 = 16 x 224 on 74 CTA pairs)
    const uint64_t rowPairs = (M + 2 * kBM - 1) / (2 * kBM), pairs = (uint64_t)SmCount() / 2;
    auto cost = [&](uint32_t bn) { uint64_t tiles = rowPairs * ((N + bn - 1) / bn); return ((tiles + pairs - 1) / pairs) * bn; };
    static const int level = [] { const char *e = getenv("HCCL_MC2_CTA_PAIR"); return e ? atoi(e) : 1; }();
    if (level >= 2 && cost(224) < cost(256)) return LaunchPlain2CtaT<224>(a, b, c, M, N, K, outFp32, s);
    return LaunchPlain2CtaT<256>(a, b, c, M, N, K, outFp32, s);
}

// HCCL_GEMM_2CTA: 0 never, otherwise (and unset) always. The CTA-pair kernel keeps the tensor pipe at 97 % of the active
// cycles against 85-88 % for the one-CTA kernel and halves the B traffic per SM. Isolated it wins clearly (1635 against 1480
// TFLOP/s on 8192 x 8192 x 4096); back to back under the board's power limit it runs at a lower clock (1140 against 1240 MHz)
// but still finishes sooner: 5.91-5.92 ms against 6.11-6.13 ms for the 8192 x 28672 x 8192 pair of the single-GPU step, two
// interleaved runs each on one box (benchmarks/gemm_sustained.py), 5.53 ms for the library GEMM on the same box.
bool Gemm2CtaEnabled(uint64_t, uint64_t, uint64_t)
{
    static const int v = [] { const char *e = getenv("HCCL_GEMM_2CTA"); return e ? atoi(e) : -1; }();
    return v != 0;
}

}  // namespace mc2
}  // namespace hccl

using namespace hccl;
using namespace hccl::mc2;

extern "C" {

// C[M,N] = A[M,K] * B[N,K]^T, bf16 operands (row-major, K contiguous), bf16 or fp32 output. K % 8 == 0, N % 8 == 0.
HcclResult HcclGemmBf16(const void *a, const void *b, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32, cudaStream_t stream)
{
    if (!a || !b || !c) return HCCL_E_PTR;
    if (m == 0 || n == 0 || k == 0 || (k % 8) || (n % 8) || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) {
        HCCL_ERROR("HcclGemmBf16: unsupported shape %llux%llux%llu (K and N must be multiples of 8)", (unsigned long long)m, (unsigned long long)n, (unsigned long long)k);
        return HCCL_E_PARA;
    }
    // narrow tiles when the problem has too few 128x256 tiles to fill the GPU
    uint64_t tiles256 = ((m + 127) / 128) * ((n + 255) / 256);
    if (Gemm2CtaEnabled(m, n, k) && tiles256 >= (uint64_t)SmCount()) return LaunchPlain2Cta(a, b, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    if (tiles256 >= (uint64_t)SmCount() || n % 256 == 0 && tiles256 * 2 > (uint64_t)SmCount()) return LaunchPlain<256>(a, b, c, m, n, k, outFp32 != 0, stream);
    uint64_t tiles128 = ((m + 127) / 128) * ((n + 127) / 128);
    if (tiles128 >= (uint64_t)SmCount() / 2) return LaunchPlain<128>(a, b, c, m, n, k, outFp32 != 0, stream);
    return LaunchPlain<64>(a, b, c, m, n, k, outFp32 != 0, stream);
}

// variant 0 = automatic choice, 1 = one-CTA tiles, 2 = 256 x 256 tiles on CTA pairs (cta_group::2)
HcclResult HcclGemmBf16Variant(const void *a, const void *b, void *c, uint64_t m, uint64_t n, uint64_t k, int outFp32, int variant, cudaStream_t stream)
{
    if (variant == 2) {
        if (!a || !b || !c) return HCCL_E_PTR;
        if (m == 0 || n == 0 || k == 0 || (k % 8) || (n % 8) || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return HCCL_E_PARA;
        return LaunchPlain2Cta(a, b, c, (uint32_t)m, (uint32_t)n, (uint32_t)k, outFp32 != 0, stream);
    }
    return HcclGemmBf16(a, b, c, m, n, k, outFp32, stream);
}

HcclResult HcclGemmCheckError(void) { return GemmCheckError(); }

uint64_t HcclGetKernelLaunchCount(void) { return KernelLaunchCounter().load(); }

}  // extern "C"
