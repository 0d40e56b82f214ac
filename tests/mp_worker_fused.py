"""Worker of the multi-GPU fused-op tests: AllGatherMatmul, MatmulReduceScatter, MatmulAllReduce over real NVLink against
an unfused NCCL + fp32 reference."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from hccl_b200.comm import init_from_env  # noqa: E402
from hccl_b200.ops import gemm, mc2, mxfp8 as mx  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def main():
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = init_from_env()
    rank, n = comm.rank, comm.size
    fails = []
    g = torch.Generator(device="cuda").manual_seed(77 + rank)
    for it, (m_local, N, K) in enumerate([(128, 256, 512), (256, 1024, 1024), (1024, 3584, 8192), (256, 1024, 1024)]):
        a = torch.randn(m_local, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        gathered = torch.empty(n * m_local, K, dtype=torch.bfloat16, device="cuda")
        out = mc2.all_gather_matmul(comm, a, w, gathered=gathered)
        torch.cuda.synchronize()
        full = torch.empty(n * m_local, K, dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(full, a)
        ref = full.float() @ w.float().t()
        if rel(out, ref) > 2e-2 or not torch.equal(gathered, full):
            fails.append(f"agmm {m_local}x{N}x{K} rel={rel(out, ref):.4f} gathered_ok={torch.equal(gathered, full)}")
    for it, (M, N, K) in enumerate([(128 * n, 256, 256), (512 * n, 1024, 512), (8192, 8192, 3584 // 2), (256 * n, 520, 256)]):
        a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        out = mc2.matmul_reduce_scatter(comm, a, w)
        torch.cuda.synchronize()
        partial = (a.float() @ w.float().t()).to(torch.bfloat16).float()
        dist.all_reduce(partial)
        rows = M // n
        r = rel(out, partial[rank * rows:(rank + 1) * rows])
        if r > 1e-2:
            fails.append(f"mmrs {M}x{N}x{K} rel={r:.4f}")
    for it, (M, N, K) in enumerate([(128, 64 * n * 2, 256), (128, 8192, 1024), (64, 1024, 512), (128, 8192, 1024)]):
        a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        out = mc2.matmul_all_reduce(comm, a, w)
        torch.cuda.synchronize()
        partial = (a.float() @ w.float().t()).to(torch.bfloat16).float()
        dist.all_reduce(partial)
        r = rel(out, partial)
        chk = out.float().sum().reshape(1).clone()
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if r > 1e-2 or lo.item() != hi.item():
            fails.append(f"mmar {M}x{N}x{K} rel={r:.4f} identical={lo.item() == hi.item()}")
    # ---- block-scaled fp8 forms: operands quantised on this rank, references from the dequantised values
    for (m_local, N, K) in [(128, 256, 256), (1024, 3584, 8192), (256, 1024, 1024)]:
        a = mx.quantize(torch.randn(m_local, K, generator=g, device="cuda").to(torch.bfloat16))
        w = mx.quantize((torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16))
        out = mx.all_gather_matmul(comm, a, w)
        torch.cuda.synchronize()
        mine = mx.dequantize(a)
        full = torch.empty(n * m_local, K, dtype=torch.float32, device="cuda")
        dist.all_gather_into_tensor(full, mine)
        r = rel(out, full @ mx.dequantize(w).t())
        if r > 1e-2:
            fails.append(f"agmm-mxfp8 {m_local}x{N}x{K} rel={r:.4f}")
    for (M, N, K) in [(128 * n, 256, 256), (8192, 8192, 3584), (256 * n, 520, 384)]:
        a = mx.quantize(torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16))
        w = mx.quantize((torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16))
        out = mx.matmul_reduce_scatter(comm, a, w)
        torch.cuda.synchronize()
        partial = (mx.dequantize(a) @ mx.dequantize(w).t()).to(torch.bfloat16).float()
        dist.all_reduce(partial)
        rows = M // n
        r = rel(out, partial[rank * rows:(rank + 1) * rows])
        if r > 1.5e-2:
            fails.append(f"mmrs-mxfp8 {M}x{N}x{K} rel={r:.4f}")
    for (M, N, K) in [(128, 128 * n * 2, 256), (128, 8192, 1024)]:
        a = mx.quantize(torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16))
        w = mx.quantize((torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16))
        out = mx.matmul_all_reduce(comm, a, w)
        torch.cuda.synchronize()
        partial = (mx.dequantize(a) @ mx.dequantize(w).t()).to(torch.bfloat16).float()
        dist.all_reduce(partial)
        r = rel(out, partial)
        if r > 1.5e-2:
            fails.append(f"mmar-mxfp8 {M}x{N}x{K} rel={r:.4f}")
    gemm.check_error()
    ok = comm.async_error() == 0
    comm.destroy()
    dist.destroy_process_group()
    if fails or not ok:
        print(f"[rank {rank}] FAIL {fails} async_ok={ok}", flush=True)
        sys.exit(1)
    if rank == 0:
        print(f"all fused multi-GPU checks passed on {n} ranks", flush=True)


if __name__ == "__main__":
    main()
