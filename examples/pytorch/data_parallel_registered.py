"""Data parallelism over a bare Communicator: gradient buckets live in registered windows of the symmetric heap and are reduced
in place by the zero-copy all-reduce kernels while the backward pass is still running.

    torchrun --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 examples/pytorch/data_parallel_registered.py

Also shows the torch memory pool whose segments are registered blocks: ordinary tensors created under it need no staging
copy either. Every rank has to allocate the same tensors in the same order inside the pool.
"""
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from hccl_b200.comm import init_from_env  # noqa: E402
from hccl_b200.parallel.data_parallel import DataParallel  # noqa: E402


def main():
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    comm = init_from_env()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(1024, 4096), nn.GELU(), nn.Linear(4096, 1024)).cuda().to(torch.bfloat16)
    dp = DataParallel(model, comm, bucket_mb=8.0)            # buckets: comm.sym_tensor windows; the all-reduce is capped at 16 CTAs
    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    torch.manual_seed(100 + comm.rank)
    for step in range(3):
        x = torch.randn(64, 1024, device="cuda", dtype=torch.bfloat16)
        opt.zero_grad(set_to_none=False)                     # keep the gradients: they are views of the buckets
        model(x).float().pow(2).mean().backward()
        dp.finish()
        opt.step()
    # parameters stay identical on every rank
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    comm.broadcast(ref, 0)
    torch.cuda.synchronize()
    assert torch.equal(flat, ref), "ranks diverged"

    pool = comm.mem_pool()
    with torch.cuda.use_mem_pool(pool):
        t = torch.full((4 << 20,), float(comm.rank + 1), device="cuda")
    comm.all_reduce(t, t)
    torch.cuda.synchronize()
    assert torch.all(t == comm.size * (comm.size + 1) / 2)
    if comm.rank == 0:
        print(f"data-parallel sample passed on {comm.size} ranks; last algorithm: {comm.last_algorithm()}", flush=True)
    del t, pool
    dp.close()
    comm.destroy()


if __name__ == "__main__":
    main()
