"""End-to-end training step of a Llama-3-architecture decoder, tensor-parallel or data-parallel, ours vs NCCL+cuBLAS.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/train_llama.py --parallel tp --impl ours
    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/train_llama.py --parallel tp --impl nccl
    torchrun ... benchmarks/train_llama.py --parallel dp --impl ours      # bucketed gradient all-reduce overlapped with backward

`--impl ours` runs every linear as a fused matmul+collective kernel (forward and backward) over this library's
communicator; `--impl nccl` runs the identical model with cuBLAS matmuls and torch.distributed (NCCL) collectives.
Synthetic tokens, random-init weights, bf16 parameters, fused AdamW. Each step includes the host-to-device copy of the
token batch from pinned memory and a device-to-host read of the loss. Prints one JSON line (rank 0): tokens/s over the
whole job, device-timed, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from hccl_b200.models.llama import Llama, LlamaConfig  # noqa: E402


class TorchDistComm:
    """The subset of the Communicator interface the model uses, on torch.distributed (baseline arm)."""

    fused = False          # tensor_parallel: use cuBLAS + these collectives instead of the fused kernels

    def __init__(self, group=None, solo: bool = False):
        self.group = group
        self.size = 1 if solo else dist.get_world_size(group)
        self.rank = 0 if solo else dist.get_rank(group)

    def all_gather(self, send, recv, stream=None):
        if self.size == 1:
            recv.view(-1).copy_(send.view(-1))
            return
        dist.all_gather_into_tensor(recv, send, group=self.group)

    def reduce_scatter(self, send, recv, op=None, stream=None):
        if self.size == 1:
            recv.view(-1).copy_(send.view(-1))
            return
        dist.reduce_scatter_tensor(recv, send, group=self.group)

    def all_reduce(self, send, recv=None, op=None, stream=None):
        from hccl_b200.types import ReduceOp
        t = send if recv is None else recv
        if recv is not None and recv.data_ptr() != send.data_ptr():
            recv.copy_(send)
        if self.size == 1:
            return
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == ReduceOp.MAX else dist.ReduceOp.SUM, group=self.group)

    def synchronize(self):
        pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--parallel", choices=["tp", "dp"], default="tp")
    ap.add_argument("--impl", choices=["ours", "ours-ddp", "nccl"], default="ours",
                    help="ours-ddp (data parallel only): torch DistributedDataParallel over this library's process-group backend")
    ap.add_argument("--model", choices=["llama3-8b", "small", "tiny"], default="llama3-8b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (reported in the config)")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bucket-mb", type=float, default=32.0)
    ap.add_argument("--dp-ctas", type=int, default=-1, help="data parallel, --impl ours: cap on the CTAs of the gradient all-reduce kernels (-1 = library default)")
    ap.add_argument("--native-gemm", action="store_true", help="data parallel: run the (collective-free) linears on this library's GEMM instead of cuBLAS")
    ap.add_argument("--staged-buckets", action="store_true", help="data parallel, --impl ours: keep the gradient buckets in ordinary device "
                    "memory instead of registered windows (set HCCL_SYM_HEAP_MB above the gradient size for registered buckets)")
    a = ap.parse_args()

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    cfg = {"llama3-8b": LlamaConfig.llama3_8b(), "small": LlamaConfig(32000, 2048, 8, 16, 8, 5632), "tiny": LlamaConfig.tiny()}[a.model]
    if a.layers:
        cfg.layers = a.layers
    tp = world if a.parallel == "tp" else 1
    dp = world // tp

    from hccl_b200.comm import Communicator, get_root_info, init_from_env
    if a.impl == "ours-ddp" and a.parallel != "dp":
        raise SystemExit("--impl ours-ddp needs --parallel dp")
    native = a.impl != "nccl"
    world_comm = init_from_env() if a.impl == "ours" else None
    if a.parallel == "tp":
        comm = world_comm if native else TorchDistComm()
    else:
        comm = Communicator.from_root_info(1, get_root_info(), 0) if native else TorchDistComm(solo=True)

    from hccl_b200.parallel import tensor_parallel
    # tensor parallel: every linear is a fused matmul + collective kernel of this library. Data parallel: the linears have no
    # collective attached, so they are plain library GEMMs (cuBLAS, as in the baseline arm) unless --native-gemm asks for this
    # library's tcgen05 GEMM; what differs between the arms is the gradient all-reduce.
    tensor_parallel.use_native_gemm(native and (a.parallel == "tp" or a.native_gemm))
    model = Llama(cfg, comm, dtype=torch.bfloat16, device=dev, seed=None)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.1, fused=True)
    dpw, grp = None, None
    if a.parallel == "dp" and world > 1:
        if a.impl == "ours":
            from hccl_b200.parallel.data_parallel import DataParallel
            dpw = DataParallel(model, world_comm, bucket_mb=a.bucket_mb, registered=not a.staged_buckets, **({} if a.dp_ctas < 0 else {"max_ctas": a.dp_ctas}))
        elif a.impl == "ours-ddp":
            os.environ.setdefault("HCCL_MAX_CTAS", "16")   # as DataParallel does: few CTAs for a collective that overlaps the backward pass
            import hccl_b200.parallel  # noqa: F401  (registers the "hccl" backend)
            grp = dist.new_group(backend="hccl")
            dist.all_reduce(torch.zeros(1, device=dev), group=grp)      # creates the group's CUDA communicator
            from contextlib import nullcontext

            from hccl_b200.parallel import process_group as hpg
            ddp_pool = None if a.staged_buckets else hpg.mem_pool()     # DDP's gradient buckets become registered windows
            with (torch.cuda.use_mem_pool(ddp_pool) if ddp_pool is not None else nullcontext()):
                model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=a.bucket_mb, gradient_as_bucket_view=True,
                                                                  process_group=grp)
        else:
            model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=a.bucket_mb, gradient_as_bucket_view=True)

    B, S = a.micro_batch, a.seq
    g = torch.Generator().manual_seed(1000 + (rank if a.parallel == "dp" else 0))     # TP ranks see the same batch
    host_tok = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory() for _ in range(4)]
    loss_host = torch.zeros(1, pin_memory=True)

    def step(i):
        tok = host_tok[i % 4].to(dev, non_blocking=True)
        loss = model(tok[:, :-1], tok[:, 1:].contiguous())
        loss.backward()
        inner = model.module if hasattr(model, "module") else model
        inner.sync_replicated_grads()
        if dpw is not None:
            dpw.finish()
        opt.step()
        opt.zero_grad(set_to_none=False)
        loss_host.copy_(loss.detach().float().reshape(1), non_blocking=True)

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tokens = B * S * dp
    if rank == 0:
        tps = tokens / (ms.item() / 1e3)
        print(json.dumps({"metric": "training tokens/s", "impl": a.impl, "parallel": f"{a.parallel}{world}", "model": a.model, "layers": cfg.layers,
                          "params": cfg.param_count(), "seq": S, "micro_batch": B, "ms_per_step": round(ms.item(), 3), "tokens_per_s": round(tps, 1),
                          "model_tflops_per_gpu": round(cfg.flops_per_token(S) * tps / world / 1e12, 1), "loss": round(float(loss_host.item()), 4),
                          "h2d_bytes_per_step": host_tok[0].numel() * 8, "d2h_bytes_per_step": 4}), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    if world_comm is not None:
        if dpw is not None:
            dpw.close()
        world_comm.destroy()
    # the DistributedDataParallel wrapper keeps its process group alive: let go of it before the groups are destroyed, so that no
    # communicator outlives the CUDA context at interpreter exit
    del opt, model
    if a.impl == "ours-ddp":
        dist.destroy_process_group(grp)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
