// MoE dispatch / combine kernels (sm_100a). One cooperative launch per direction; see include/hccl/hccl_moe.h.
#pragma once
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "../kernels/primitives.cuh"

namespace hccl {
namespace moe {

namespace cg = cooperative_groups;
using namespace dev;

constexpr int kMoeThreads = 512;
constexpr int kMaxExperts = 320;

// Offsets (bytes) inside the per-rank symmetric workspace.
struct MoeLayout {
    uint64_t recvX, recvScales, recvSrc, yBuf, recvCounts, pos, slotMap, cntCta, baseSend, total;
};

struct MoeArgs {
    const void *x;             // [T, H] bf16
    const int32_t *topkIdx;    // [T, K]
    const float *weights;      // [T, K] (combine)
    void *out;                 // [T, H] bf16 (combine)
    uint32_t T, K, H, E, cap, mxfp8;
    uint64_t wsOff;            // workspace offset in every heap
    MoeLayout L;
    uint32_t identity;         // emulation: copy recvX -> yBuf at the end of dispatch
};

__device__ __forceinline__ KCtx MoeEnter(const DevComm *c, uint32_t chan)
{
    KCtx k;
#ifdef HCCL_DEBUG_BOUNDS
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) g_boundsComm = c;
#endif
    k.c = c; k.rank = c->rank; k.nranks = c->nranks; k.heap = c->heap[c->rank];
    k.ctrl = CtrlOf(k.heap); k.flags = FlagsOf(k.heap);
    k.half = 0; k.chan = chan; k.syncs = 0; k.ok = true; k.vGrid = gridDim.x; k.vBlock = blockIdx.x; k.cclShift = 0; k.seq = 0xffffffffu;   // not counted by the op counter: no trace record
    k.epoch = LdVolatile(&k.ctrl->chanEpoch[chan]);
    return k;
}
__device__ __forceinline__ void MoeLeave(KCtx &k)
{
    __syncthreads();
    if (threadIdx.x == 0) *((volatile uint32_t *)&k.ctrl->chanEpoch[k.chan]) = k.epoch + k.syncs;
}

// e8m0 scale for a block with absolute maximum `amax`: the smallest power of two s with amax / s <= 448
__device__ __forceinline__ uint8_t E8m0For(float amax)
{
    if (amax <= 0.f) return 127 - 8;
    int e;
    float m = frexpf(amax / 448.f, &e);     // amax/448 = m * 2^e, m in [0.5, 1)
    if (m == 0.5f) e -= 1;
    int biased = e + 127;
    return (uint8_t)(biased < 0 ? 0 : biased > 254 ? 254 : biased);
}
__device__ __forceinline__ uint8_t ToE4m3(float v)
{
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

template <bool EMU>
__global__ void __launch_bounds__(kMoeThreads) MoeDispatchKernel(const DevComm *comms, const __grid_constant__ MoeArgs av, const MoeArgs *emuArgs)
{
    const DevComm *c = EMU ? &comms[blockIdx.y] : comms;
    const MoeArgs &A = EMU ? emuArgs[blockIdx.y] : av;
    cg::grid_group grid = cg::this_grid();
    const int n = c->nranks, me = c->rank;
    char *ws = c->heap[me] + A.wsOff;
    const uint32_t E = A.E, EL = E / n, entries = A.T * A.K;
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    uint32_t *pos = (uint32_t *)(ws + A.L.pos);
    uint64_t *slotMap = (uint64_t *)(ws + A.L.slotMap);
    uint32_t *cntCta = (uint32_t *)(ws + A.L.cntCta);
    uint32_t *baseSend = (uint32_t *)(ws + A.L.baseSend);
    int32_t *recvCounts = (int32_t *)(ws + A.L.recvCounts);
    const uint32_t per = (entries + G - 1) / G, lo = cta * per, hi = lo + per < entries ? lo + per : entries;

    // 1. per-CTA histogram and in-CTA ordinals (thread e walks the chunk: deterministic order)
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
        uint32_t cnt = 0;
        for (uint32_t i = lo; i < hi; ++i)
            if ((uint32_t)A.topkIdx[i] == e) pos[i] = cnt++;
        cntCta[cta * E + e] = cnt;
    }
    __threadfence();
    grid.sync();

    // 2. CTA 0 publishes this rank's per-expert totals to every rank and waits for everyone's
    KCtx k = MoeEnter(c, 0);
    if (cta == 0) {
        for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
            uint32_t tot = 0;
            for (uint32_t g = 0; g < G; ++g) tot += cntCta[g * E + e];
            for (int r = 0; r < n; ++r) FlagsOf(c->heap[r])->moeCount[me][e] = tot;
        }
        ChannelBarrier(k, 61);
        // my base row at the destination of expert e: rows of earlier experts of that rank + rows of earlier sources
        for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
            const uint32_t d = e / EL, first = d * EL;
            uint32_t base = 0;
            for (uint32_t e2 = first; e2 < e; ++e2)
                for (int s = 0; s < n; ++s) base += k.flags->moeCount[s][e2];
            for (int s = 0; s < me; ++s) base += k.flags->moeCount[s][e];
            baseSend[e] = base;
        }
        for (uint32_t le = threadIdx.x; le < EL; le += blockDim.x) {
            uint32_t tot = 0;
            for (int s = 0; s < n; ++s) tot += k.flags->moeCount[s][me * EL + le];
            recvCounts[le] = (int32_t)tot;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t rows = 0;
            for (uint32_t le = 0; le < EL; ++le) rows += (uint32_t)recvCounts[le];
            if (rows > A.cap) {     // receive buffer too small: report, move nothing
                DevStatus *st = c->status;
                st->rank = (uint32_t)me; st->observed = rows; st->expected = A.cap; st->phase = 62;
                __threadfence_system();
                *((volatile uint32_t *)&st->code) = 2u;
            }
        }
        __threadfence();
    }
    grid.sync();
    // every rank checks every destination's load against the capacity (same numbers everywhere -> same decision)
    bool overflow = false;
    for (int d = 0; d < n && !overflow; ++d) {
        uint32_t rows = 0;
        for (uint32_t le = 0; le < EL; ++le)
            for (int s = 0; s < n; ++s) rows += k.flags->moeCount[s][d * EL + le];
        overflow = rows > A.cap;
    }

    // 3. scatter: one warp per (token, k) row
    if (!overflow) {
        __shared__ uint32_t sCtaBase[kMaxExperts];
        for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
            uint32_t b = 0;
            for (uint32_t g = 0; g < cta; ++g) b += cntCta[g * E + e];
            sCtaBase[e] = b;
        }
        __syncthreads();
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
        const uint32_t rowBytes = A.H * 2;
        for (uint32_t i = lo + warp; i < hi; i += warps) {
            const uint32_t e = (uint32_t)A.topkIdx[i], t = i / A.K, d = e / EL;
            const uint32_t row = baseSend[e] + sCtaBase[e] + pos[i];
            char *dws = c->heap[d] + A.wsOff;
            if (!HCCL_RANGE_OK(dws + A.L.recvX + (uint64_t)row * (A.mxfp8 ? A.H : rowBytes), A.mxfp8 ? A.H : rowBytes)) continue;
            const uint4 *src = (const uint4 *)((const char *)A.x + (uint64_t)t * rowBytes);
            if (!A.mxfp8) {
                uint4 *dst = (uint4 *)(dws + A.L.recvX + (uint64_t)row * rowBytes);
                for (uint32_t v = lane; v < rowBytes / 16; v += 32 * 4) {
                    uint4 r0 = src[v], r1, r2, r3;
                    const bool b1 = v + 32 < rowBytes / 16, b2 = v + 64 < rowBytes / 16, b3 = v + 96 < rowBytes / 16;
                    if (b1) r1 = src[v + 32];
                    if (b2) r2 = src[v + 64];
                    if (b3) r3 = src[v + 96];
                    dst[v] = r0;
                    if (b1) dst[v + 32] = r1;
                    if (b2) dst[v + 64] = r2;
                    if (b3) dst[v + 96] = r3;
                }
            } else {
                // each lane quantises blocks of 32 values: 64 bytes in, 32 bytes + 1 scale byte out
                uint8_t *dq = (uint8_t *)(dws + A.L.recvX + (uint64_t)row * A.H);
                uint8_t *ds = (uint8_t *)(dws + A.L.recvScales + (uint64_t)row * (A.H / 32));
                for (uint32_t b = lane; b < A.H / 32; b += 32) {
                    uint4 raw[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) raw[q] = src[b * 4 + q];
                    const __nv_bfloat16 *h = (const __nv_bfloat16 *)raw;
                    float f[32], amax = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) { f[j] = __bfloat162float(h[j]); amax = fmaxf(amax, fabsf(f[j])); }
                    const uint8_t se = E8m0For(amax);
                    const float inv = exp2f((float)(127 - (int)se));
                    uint4 o[2];
                    uint8_t *ob = (uint8_t *)o;
#pragma unroll
                    for (int j = 0; j < 32; ++j) ob[j] = ToE4m3(f[j] * inv);
                    ((uint4 *)(dq + b * 32))[0] = o[0];
                    ((uint4 *)(dq + b * 32))[1] = o[1];
                    ds[b] = se;
                }
            }
            if (lane == 0) {
                ((int32_t *)(dws + A.L.recvSrc))[row] = (int32_t)(((uint32_t)me << 24) | t);
                slotMap[i] = ((uint64_t)d << 32) | row;
            }
        }
    }
    __threadfence_system();
    grid.sync();
    // 4. everyone has finished writing: after this barrier the received rows are visible
    if (cta == 0) {
        ChannelBarrier(k, 63);
        MoeLeave(k);
        __threadfence();
    }
    if (A.identity) {     // emulation helper: "experts" that return their input
        grid.sync();
        if (!A.mxfp8) {
            uint32_t rows = 0;
            for (uint32_t le = 0; le < EL; ++le) rows += (uint32_t)recvCounts[le];
            Part p = PartOf((uint64_t)rows * A.H * 2, G, cta);
            BlockCopy(ws + A.L.yBuf + p.off, ws + A.L.recvX + p.off, p.len);
        } else {
            // block-scaled payload: the stand-in expert dequantises (e4m3 value x 2^(scale - 127)) into the bf16 output buffer
            uint32_t rows = 0;
            for (uint32_t le = 0; le < EL; ++le) rows += (uint32_t)recvCounts[le];
            const uint32_t blocksPerRow = A.H / 32;
            const uint64_t blocks = (uint64_t)rows * blocksPerRow;
            for (uint64_t b = (uint64_t)cta * blockDim.x + threadIdx.x; b < blocks; b += (uint64_t)G * blockDim.x) {
                const uint8_t *q = (const uint8_t *)(ws + A.L.recvX) + b * 32;
                const float scale = exp2f((float)((int)((const uint8_t *)(ws + A.L.recvScales))[b] - 127));
                __nv_bfloat16 *y = (__nv_bfloat16 *)(ws + A.L.yBuf) + b * 32;
                for (int j = 0; j < 32; ++j) {
                    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)q[j], __NV_E4M3);
                    y[j] = __float2bfloat16(__half2float(__half(hr)) * scale);
                }
            }
        }
    }
}

template <bool EMU>
__global__ void __launch_bounds__(kMoeThreads) MoeCombineKernel(const DevComm *comms, const __grid_constant__ MoeArgs av, const MoeArgs *emuArgs)
{
    const DevComm *c = EMU ? &comms[blockIdx.y] : comms;
    const MoeArgs &A = EMU ? emuArgs[blockIdx.y] : av;
    cg::grid_group grid = cg::this_grid();
    const int me = c->rank;
    char *ws = c->heap[me] + A.wsOff;
    const uint64_t *slotMap = (const uint64_t *)(ws + A.L.slotMap);
    // every rank's expert outputs are complete once it has entered this kernel
    if (blockIdx.x == 0) {
        KCtx k = MoeEnter(c, 0);
        ChannelBarrier(k, 71);
        MoeLeave(k);
        __threadfence();
    }
    grid.sync();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const uint32_t vecPerRow = A.H / 8, K = A.K;
    for (uint32_t t = blockIdx.x * warps + warp; t < A.T; t += gridDim.x * warps) {
        const char *rows[16];
        float w[16];
        for (uint32_t kk = 0; kk < K; ++kk) {
            uint64_t s = slotMap[t * K + kk];
            rows[kk] = c->heap[(uint32_t)(s >> 32)] + A.wsOff + A.L.yBuf + (uint64_t)(uint32_t)s * A.H * 2;
            w[kk] = A.weights[t * K + kk];
        }
        uint4 *dst = (uint4 *)((char *)A.out + (uint64_t)t * A.H * 2);
        for (uint32_t v = lane; v < vecPerRow; v += 32) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (uint32_t k0 = 0; k0 < K; k0 += 8) {     // eight peer loads in flight, then accumulate in k order
                uint4 raw[8];
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) if (k0 + j < K) raw[j] = ((const uint4 *)rows[k0 + j])[v];
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    if (k0 + j >= K) break;
                    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw[j];
                    const float wk = w[k0 + j];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float2 f = __bfloat1622float2(h[q]);
                        acc[2 * q] += wk * f.x;
                        acc[2 * q + 1] += wk * f.y;
                    }
                }
            }
            uint4 o;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0], acc[1]), t1 = __floats2bfloat162_rn(acc[2], acc[3]);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4], acc[5]), t3 = __floats2bfloat162_rn(acc[6], acc[7]);
            o.x = *(uint32_t *)&t0; o.y = *(uint32_t *)&t1; o.z = *(uint32_t *)&t2; o.w = *(uint32_t *)&t3;
            dst[v] = o;
        }
    }
}

}  // namespace moe
}  // namespace hccl
