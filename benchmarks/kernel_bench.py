"""Single-GPU kernel benchmarks (also the small cases used for profiler captures).

    python benchmarks/kernel_bench.py gemm --m 8192 --n 8192 --k 4096
    python benchmarks/kernel_bench.py emu-allreduce --ranks 4 --mb 64 --alg SmAllReduceMesh1DTwoShot
    python benchmarks/kernel_bench.py emu-fused --kind 0 --ranks 2 --m 2048 --n 4096 --k 4096
    python benchmarks/kernel_bench.py emu-moe --ranks 4 --tokens 1024 --hidden 4096

`gemm` times the tcgen05 kernel against torch.matmul (cuBLAS) with CUDA events after warm-up; the `emu-*` cases run the
multi-rank kernels with every rank's CTAs in one cooperative launch on this GPU (blockIdx.y = rank), which shows their
memory traffic and instruction mix without NVLink. Each case prints one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def _time(fn, iters, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()                     # a write larger than L2 evicts the previous iteration's lines
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def bench_gemm(a):
    from hccl_b200.ops import gemm

    x = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda") if a.flush else None
    ours = _time(lambda: gemm.gemm_bf16(x, w, out=out, variant=a.variant), a.iters, flush=flush)
    gemm.check_error()
    res = {"case": "gemm", "variant": a.variant, "m": a.m, "n": a.n, "k": a.k, "ours_ms": round(ours, 4), "ours_tflops": round(2 * a.m * a.n * a.k / ours / 1e9, 1)}
    if not a.no_cublas:
        ref = torch.empty_like(out)
        cub = _time(lambda: torch.matmul(x, w.t(), out=ref), a.iters, flush=flush)
        res.update(cublas_ms=round(cub, 4), cublas_tflops=round(2 * a.m * a.n * a.k / cub / 1e9, 1),
                   max_abs_diff=float((out.float() - ref.float()).abs().max()))
    print(json.dumps(res), flush=True)


def bench_mxgemm(a):
    """Block-scaled fp8 GEMM of this library against torch._scaled_mm (cuBLASLt fp8, one scale per tensor) and bf16 cuBLAS."""
    from hccl_b200.ops import gemm, mxfp8 as mx

    x = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda") * 0.02).to(torch.bfloat16)
    qa, qw = mx.quantize(x), mx.quantize(w)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda") if a.flush else None
    ours = _time(lambda: mx.gemm(qa, qw, out=out, tile_n=a.variant), a.iters, flush=flush)
    gemm.check_error()
    quant = _time(lambda: mx.quantize(x, out=qa), a.iters, flush=flush)
    flops = 2 * a.m * a.n * a.k
    ref = mx.dequantize(qa) @ mx.dequantize(qw).t() if a.m * a.n <= (1 << 26) else None
    res = {"case": "mxgemm", "tile_n": a.variant, "m": a.m, "n": a.n, "k": a.k, "ours_ms": round(ours, 4), "ours_tflops": round(flops / ours / 1e9, 1),
           "quantize_ms": round(quant, 4)}
    if ref is not None:
        res["rel_err"] = float((out.float() - ref).abs().max() / ref.abs().max())
    if not a.no_cublas:
        one = torch.ones((), device="cuda")
        x8, w8 = x.to(torch.float8_e4m3fn), w.to(torch.float8_e4m3fn)
        o2 = torch.empty_like(out)
        t8 = _time(lambda: torch._scaled_mm(x8, w8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=o2), a.iters, flush=flush)
        t16 = _time(lambda: torch.matmul(x, w.t(), out=o2), a.iters, flush=flush)
        res.update(scaled_mm_fp8_ms=round(t8, 4), scaled_mm_fp8_tflops=round(flops / t8 / 1e9, 1), cublas_bf16_ms=round(t16, 4))
    print(json.dumps(res), flush=True)


def bench_emu_allreduce(a):
    from hccl_b200.types import ReduceOp
    from hccl_b200.utils import emu

    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[a.dtype]
    n = (a.mb << 20) // torch.empty(0, dtype=dtype).element_size()
    ins = [torch.randn(n, device="cuda").to(dtype) for _ in range(a.ranks)]
    outs = [torch.empty_like(t) for t in ins]
    with emu.EmuWorld(a.ranks, max(2 * (a.mb << 20), 8 << 20)) as w:
        def run():
            rc = w.run(2, a.alg, ins, outs, n, dtype, ReduceOp.SUM, max_ctas=a.ctas)
            assert rc == 0, rc
        ms = _time(run, a.iters, warmup=2)
        ref = torch.stack([t.float() for t in ins]).sum(0)
        err = float((outs[0].float() - ref).abs().max())
    # every rank reads all inputs once and writes its output once (two-shot: plus the scratch round trip)
    print(json.dumps({"case": "emu-allreduce", "alg": a.alg, "ranks": a.ranks, "mb_per_rank": a.mb, "dtype": a.dtype, "ms": round(ms, 4),
                      "max_abs_err": err}), flush=True)


def bench_emu_fused(a):
    from hccl_b200.utils import emu

    R = a.ranks
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)
    ctas = 148 // R
    if a.kind == 0:
        A = [mk(a.m, a.k) for _ in range(R)]
        B = [mk(a.n, a.k) for _ in range(R)]
        O = [torch.empty(R * a.m, a.n, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
        arena = 4 * R * a.m * a.k + (1 << 20)
        flops = 2 * R * a.m * a.n * a.k * R
    else:
        A = [mk(a.m, a.k) for _ in range(R)]
        B = [mk(a.n, a.k) for _ in range(R)]
        rows = a.m // R if a.kind == 1 else a.m
        O = [torch.empty(rows, a.n, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
        arena = 8 * a.m * a.n + (1 << 20)
        flops = 2 * a.m * a.n * a.k * R
    with emu.EmuWorld(R, 1 << 20, arena_bytes=arena) as w:
        def run():
            rc = w.fused(a.kind, A, B, O, a.m, a.n, a.k, ctas, comm_ctas=2)
            assert rc == 0, rc
        ms = _time(run, a.iters, warmup=2)
    print(json.dumps({"case": "emu-fused", "kind": ["allgather_matmul", "matmul_reduce_scatter", "matmul_all_reduce"][a.kind], "ranks": R,
                      "m": a.m, "n": a.n, "k": a.k, "ms": round(ms, 4), "tflops_all_ranks": round(flops / ms / 1e9, 1)}), flush=True)


def bench_emu_moe(a):
    from hccl_b200.ops import moe
    from hccl_b200.utils import emu

    l = moe._decl()
    R, T, E, K, H = a.ranks, a.tokens, a.experts, a.topk, a.hidden
    cfg = moe.HcclMoeConfig(E, K, H, T, R * T * K, 0)
    xs = [torch.randn(T, H, device="cuda").to(torch.bfloat16) for _ in range(R)]
    idxs = [torch.topk(torch.randn(T, E, device="cuda"), K, dim=1).indices.to(torch.int32).contiguous() for _ in range(R)]
    ws = [torch.rand(T, K, device="cuda").contiguous() for _ in range(R)]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    arr = lambda ts: (ctypes.c_void_p * R)(*[t.data_ptr() for t in ts])
    with emu.EmuWorld(R, 1 << 20, arena_bytes=4 * R * T * K * H * 2 + (8 << 20)) as w:
        def run():
            rc = l.HcclEmuMoeRoundTrip(w._h, ctypes.byref(cfg), arr(xs), arr(idxs), arr(ws), arr(outs), T, None, max(1, min(16, 148 // R)))
            torch.cuda.synchronize()
            assert rc == 0, rc
        ms = _time(run, a.iters, warmup=2)
    moved = 2 * R * T * K * H * 2    # dispatch + combine, bf16
    print(json.dumps({"case": "emu-moe", "ranks": R, "tokens_per_rank": T, "experts": E, "topk": K, "hidden": H, "ms": round(ms, 4),
                      "gb_moved": round(moved / 1e9, 3)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192); g.add_argument("--n", type=int, default=8192); g.add_argument("--k", type=int, default=4096)
    g.add_argument("--iters", type=int, default=10); g.add_argument("--flush", action="store_true"); g.add_argument("--no-cublas", action="store_true")
    g.add_argument("--variant", type=int, default=0, help="0 auto, 1 one-CTA tiles, 2 CTA-pair 256x256 tiles")
    x = sub.add_parser("mxgemm")
    x.add_argument("--m", type=int, default=8192); x.add_argument("--n", type=int, default=8192); x.add_argument("--k", type=int, default=4096)
    x.add_argument("--iters", type=int, default=10); x.add_argument("--flush", action="store_true"); x.add_argument("--no-cublas", action="store_true")
    x.add_argument("--variant", type=int, default=0, help="tile width: 0 auto, 128, 192, 256")
    r = sub.add_parser("emu-allreduce")
    r.add_argument("--ranks", type=int, default=4); r.add_argument("--mb", type=int, default=64); r.add_argument("--dtype", default="fp32")
    r.add_argument("--alg", default="SmAllReduceMesh1DTwoShot"); r.add_argument("--ctas", type=int, default=32); r.add_argument("--iters", type=int, default=5)
    f = sub.add_parser("emu-fused")
    f.add_argument("--kind", type=int, default=0); f.add_argument("--ranks", type=int, default=2); f.add_argument("--m", type=int, default=2048)
    f.add_argument("--n", type=int, default=4096); f.add_argument("--k", type=int, default=4096); f.add_argument("--iters", type=int, default=5)
    m = sub.add_parser("emu-moe")
    m.add_argument("--ranks", type=int, default=4); m.add_argument("--tokens", type=int, default=1024); m.add_argument("--experts", type=int, default=64)
    m.add_argument("--topk", type=int, default=8); m.add_argument("--hidden", type=int, default=4096); m.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    {"gemm": bench_gemm, "mxgemm": bench_mxgemm, "emu-allreduce": bench_emu_allreduce, "emu-fused": bench_emu_fused, "emu-moe": bench_emu_moe}[a.case](a)


if __name__ == "__main__":
    main()
