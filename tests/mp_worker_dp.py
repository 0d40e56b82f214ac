"""Worker for the data-parallel GPU test: every rank holds the same model, sees its slice of one batch, and must end up with
the gradient of the whole batch; buckets live in registered windows (reduced in place by the zero-copy kernels) or in
ordinary device memory (staged)."""
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from hccl_b200.comm import init_from_env  # noqa: E402
from hccl_b200.parallel.data_parallel import DataParallel  # noqa: E402


def model(dev):
    torch.manual_seed(3)
    return nn.Sequential(nn.Linear(256, 1024), nn.Tanh(), nn.Linear(1024, 1024), nn.Tanh(), nn.Linear(1024, 16)).to(dev)


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda")
    comm = init_from_env()
    world = comm.size
    per = 8
    torch.manual_seed(0)
    x, y = torch.randn(per * world, 256, device=dev), torch.randn(per * world, 16, device=dev)
    ref = model(dev)
    ((ref(x) - y) ** 2).mean().backward()
    want = [p.grad.clone() for p in ref.parameters()]
    fails = []
    for registered, bucket_mb in ((True, 8.0), (True, 0.5), (False, 0.5)):
        m = model(dev)
        dp = DataParallel(m, comm, bucket_mb=bucket_mb, registered=registered)
        for step in range(3):                                # later steps reuse the buckets
            m.zero_grad(set_to_none=(step == 2))             # steps 0-1: gradients accumulate straight into the buckets; step 2: copied in
            ((m(x[rank * per:(rank + 1) * per]) - y[rank * per:(rank + 1) * per]) ** 2).mean().backward()
            dp.finish()
            torch.cuda.synchronize()
            for g, w in zip((p.grad for p in m.parameters()), want):
                if not torch.allclose(g, w, atol=1e-5, rtol=1e-4):
                    fails.append((registered, bucket_mb, step, float((g - w).abs().max())))
        alg = comm.last_algorithm()
        # the 8 MB bucket holds the 4 MB middle layer: large enough for the zero-copy rule unless an explicit request overrides it
        if registered and bucket_mb == 8.0 and "HCCL_ALGO_NAME" not in os.environ and "HCCL_OP_EXPANSION_MODE" not in os.environ:
            if not any(b.numel * 4 >= (1 << 20) for b in dp.buckets):
                fails.append(("no bucket above 1 MB", len(dp.buckets)))
        if rank == 0:
            print(f"registered={registered} bucket_mb={bucket_mb}: {len(dp.buckets)} buckets, {dp.launched} launches, last algorithm {alg}", flush=True)
        dp.close()
    comm.barrier()
    torch.cuda.synchronize()
    if comm.async_error() != 0:
        fails.append("async error")
    comm.destroy()
    if fails:
        print(f"[rank {rank}] failures: {fails[:6]}", flush=True)
        sys.exit(1)
    if rank == 0:
        print(f"data-parallel checks passed on {world} ranks", flush=True)


if __name__ == "__main__":
    main()
