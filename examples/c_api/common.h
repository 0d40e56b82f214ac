// Shared scaffolding of the C API samples: one thread per rank in this process, root info created once and handed to
// every thread, buffers in device memory on a CUDA communicator or in host memory on the simulation backend
// (HCCL_BACKEND=sim runs every sample on a machine without GPUs).
//
// The samples follow the shape of HCCL's (reference: examples/02_collectives/01_allreduce/main.cc:44-148: device count ->
// root info -> one thread per device -> HcclCommInitRootInfo -> operator -> synchronize -> check -> destroy).
#pragma once
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <strings.h>
#include <thread>
#include <vector>
#include "hccl/hccl.h"
#include "hccl/hccl_dfx.h"

#define HCCLCHECK(call)                                                                                         \
    do {                                                                                                        \
        HcclResult _r = (call);                                                                                 \
        if (_r != HCCL_SUCCESS) {                                                                               \
            fprintf(stderr, "%s:%d %s -> %d (%s)\n", __FILE__, __LINE__, #call, (int)_r, HcclGetErrorString(_r)); \
            exit(1);                                                                                            \
        }                                                                                                       \
    } while (0)
#define CUDACHECK(call)                                                                                 \
    do {                                                                                                \
        cudaError_t _e = (call);                                                                        \
        if (_e != cudaSuccess) {                                                                        \
            fprintf(stderr, "%s:%d %s -> %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(_e));     \
            exit(1);                                                                                    \
        }                                                                                               \
    } while (0)

struct RankCtx {
    uint32_t rank = 0, size = 0;
    HcclComm comm = nullptr;
    bool cuda = false;
    cudaStream_t stream = nullptr;

    void *Alloc(size_t bytes) const
    {
        void *p = nullptr;
        if (cuda) CUDACHECK(cudaMalloc(&p, bytes ? bytes : 1));
        else p = malloc(bytes ? bytes : 1);
        return p;
    }
    void Free(void *p) const
    {
        if (cuda) cudaFree(p);
        else free(p);
    }
    void Upload(void *dst, const void *src, size_t bytes) const
    {
        if (cuda) CUDACHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
        else memcpy(dst, src, bytes);
    }
    void Download(void *dst, const void *src, size_t bytes) const
    {
        if (cuda) CUDACHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
        else memcpy(dst, src, bytes);
    }
    // Waits for everything enqueued so far (stream on CUDA, worker queue on the simulation backend).
    void Sync() const
    {
        if (cuda) CUDACHECK(cudaStreamSynchronize(stream));
        else HCCLCHECK(HcclSimStreamSynchronize(comm));
    }
};

inline bool WantSim()
{
    const char *e = getenv("HCCL_BACKEND");
    if (e && (!strcasecmp(e, "sim") || !strcasecmp(e, "host"))) return true;
    int n = 0;
    return cudaGetDeviceCount(&n) != cudaSuccess || n == 0;
}

// Runs body(ctx) on `nranks` threads (default: one per visible GPU, or EXAMPLE_RANKS / 4 on the simulation backend).
inline int RunRanks(const std::function<bool(RankCtx &)> &body, int nranks = 0)
{
    const bool sim = WantSim();
    if (nranks == 0) {
        if (const char *e = getenv("EXAMPLE_RANKS")) nranks = atoi(e);
        if (nranks <= 0) {
            if (sim) nranks = 4;
            else CUDACHECK(cudaGetDeviceCount(&nranks));
        }
    }
    HcclRootInfo root;
    HCCLCHECK(HcclGetRootInfo(&root));
    std::vector<std::thread> th;
    std::vector<int> ok(nranks, 0);
    for (int r = 0; r < nranks; ++r)
        th.emplace_back([&, r] {
            RankCtx ctx;
            ctx.rank = (uint32_t)r;
            ctx.size = (uint32_t)nranks;
            HcclCommConfig cfg;
            HcclCommConfigInit(&cfg);
            cfg.hcclBackend = sim ? 1 : 2;
            if (!sim) CUDACHECK(cudaSetDevice(r));
            HCCLCHECK(HcclCommInitRootInfoConfig((uint32_t)nranks, &root, (uint32_t)r, &cfg, &ctx.comm));
            ctx.cuda = HcclCommIsCuda(ctx.comm) != 0;
            if (ctx.cuda) CUDACHECK(cudaStreamCreate(&ctx.stream));
            ok[r] = body(ctx) ? 1 : 0;
            ctx.Sync();
            HCCLCHECK(HcclCommDestroy(ctx.comm));
            if (ctx.cuda) cudaStreamDestroy(ctx.stream);
        });
    for (auto &t : th) t.join();
    int good = 0;
    for (int v : ok) good += v;
    printf("%s: %d/%d ranks passed (%s backend)\n", good == nranks ? "PASS" : "FAIL", good, nranks, sim ? "simulation" : "CUDA");
    return good == nranks ? 0 : 1;
}
