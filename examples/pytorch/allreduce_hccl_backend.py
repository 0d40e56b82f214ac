"""torch.distributed with backend "hccl": all-reduce, broadcast and a DDP step.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/pytorch/allreduce_hccl_backend.py
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/pytorch/allreduce_hccl_backend.py --cpu

The counterpart of HCCL's framework sample (reference: examples/03_ai_framework/01_pytorch/hccl_pytorch_allreduce_test.py:19-55,
which initialises torch.distributed with backend="hccl" through torch_npu). CUDA tensors run on the NVLink kernels, CPU
tensors on the host simulation backend, so `--cpu` works on a machine without GPUs.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import hccl_b200.parallel  # noqa: F401,E402  (registers the "hccl" backend)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if a.cpu:
        dev = torch.device("cpu")
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("hccl", rank=rank, world_size=world)

    x = torch.full((1 << 20,), float(rank + 1), device=dev)
    dist.all_reduce(x)
    assert torch.all(x == world * (world + 1) / 2)

    b = torch.arange(1000, device=dev, dtype=torch.float32) * (rank + 1)
    dist.broadcast(b, src=world - 1)
    assert torch.equal(b, torch.arange(1000, device=dev, dtype=torch.float32) * world)

    torch.manual_seed(0)
    model = torch.nn.Linear(256, 256).to(dev)
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=None if a.cpu else [dev.index])
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
    torch.manual_seed(100 + rank)
    loss = ddp(torch.randn(32, 256, device=dev)).square().mean()
    loss.backward()                                   # gradients are averaged by bucketed all-reduces on the "hccl" backend
    opt.step()
    w = model.weight.detach().clone()
    ref = w.clone()
    dist.broadcast(ref, src=0)
    assert torch.allclose(w, ref), "replicas diverged"
    if not a.cpu:
        torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print(f"hccl backend sample passed on {world} ranks ({dev.type})", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
