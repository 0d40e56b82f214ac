"""A tensor + sequence parallel SwiGLU MLP whose linears are the fused matmul+collective kernels (forward and backward).

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/pytorch/tensor_parallel_mlp.py

Each rank holds 1/tp of the gate/up and down projections and 1/tp of the tokens; AllGather->matmul and
matmul->ReduceScatter each run as ONE sm_100a kernel over the communicator's symmetric heap.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from hccl_b200.comm import init_from_env  # noqa: E402
from hccl_b200.parallel.tensor_parallel import TensorParallelMLP  # noqa: E402


def main():
    comm = init_from_env()
    tp, rank = comm.size, comm.rank
    hidden, ffn, tokens = 4096, 14336, 8192
    mlp = TensorParallelMLP(comm, hidden, ffn, device="cuda", seed=1)
    x = torch.randn(tokens // tp, hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    for _ in range(3):
        y = mlp(x)
        y.float().square().mean().backward()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        y = mlp(x)
        y.float().square().mean().backward()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / 10
    flops = 6 * tokens * hidden * ffn * 3 / tp
    if rank == 0:
        print(f"TP={tp} MLP fwd+bwd {ms:.3f} ms/step, {flops / ms / 1e9:.0f} TFLOP/s per GPU", flush=True)
    comm.destroy()


if __name__ == "__main__":
    main()
