// One call creates the communicators of every device of this process (HcclCommInitAll); each is then driven from its own
// thread. With HCCL_BACKEND=sim the same call creates simulated ranks.
#include "common.h"

int main()
{
    const bool sim = WantSim();
    int n = 0;
    if (const char *e = getenv("EXAMPLE_RANKS")) n = atoi(e);
    if (n <= 0) {
        if (sim) n = 4;
        else CUDACHECK(cudaGetDeviceCount(&n));
    }
    if (sim) setenv("HCCL_BACKEND", "sim", 1);
    std::vector<int32_t> devices(n);
    for (int i = 0; i < n; ++i) devices[i] = i;
    std::vector<HcclComm> comms(n, nullptr);
    HCCLCHECK(HcclCommInitAll((uint32_t)n, devices.data(), comms.data()));
    std::vector<int> ok(n, 0);
    std::vector<std::thread> th;
    for (int r = 0; r < n; ++r)
        th.emplace_back([&, r] {
            RankCtx c;
            c.rank = (uint32_t)r; c.size = (uint32_t)n; c.comm = comms[r];
            c.cuda = HcclCommIsCuda(c.comm) != 0;
            if (c.cuda) { CUDACHECK(cudaSetDevice(r)); CUDACHECK(cudaStreamCreate(&c.stream)); }
            uint32_t id = 99, sz = 0;
            HCCLCHECK(HcclGetRankId(c.comm, &id));
            HCCLCHECK(HcclGetRankSize(c.comm, &sz));
            const uint64_t count = 10000;
            std::vector<float> host(count, (float)(r + 1));
            void *buf = c.Alloc(count * 4);
            c.Upload(buf, host.data(), count * 4);
            HCCLCHECK(HcclAllReduce(buf, buf, count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, c.comm, c.stream));
            c.Sync();
            c.Download(host.data(), buf, count * 4);
            c.Free(buf);
            bool good = id == (uint32_t)r && sz == (uint32_t)n;
            for (float v : host) good = good && v == (float)(n * (n + 1) / 2);
            ok[r] = good ? 1 : 0;
            c.Sync();
            HCCLCHECK(HcclCommDestroy(c.comm));
            if (c.cuda) cudaStreamDestroy(c.stream);
        });
    for (auto &t : th) t.join();
    int good = 0;
    for (int v : ok) good += v;
    printf("%s: %d/%d ranks passed (%s backend)\n", good == n ? "PASS" : "FAIL", good, n, sim ? "simulation" : "CUDA");
    return good == n ? 0 : 1;
}
