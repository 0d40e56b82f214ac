"""Headline benchmark: fused GEMM + collective TFLOP/s on the Llama-3-70B MLP shapes under tensor parallelism.

One step = the two tensor-parallel GEMMs of the MLP with their collectives:
    h   = AllGather_rows(x_local[8192/N, 8192]) @ W_up[28672/N, 8192]^T          -> [8192, 28672/N]
    out = ReduceScatter_rows(h[8192, 28672/N] @ W_down[8192, 28672/N]^T)          -> [8192/N, 8192]
The problem is fixed as N grows (strong scaling); at N = 8 the per-rank shapes are exactly the configured ones; at N = 1 the
collectives vanish and the step is two GEMMs. `value` is the whole-job TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--dtype bf16|mxfp8] [--repeats R]
For N > 1 launch through torchrun:  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1
    --master-port P bench.py --gpus N --steps K --warmup W

--impl ours       each half of the step is ONE fused sm_100a kernel of this library (tcgen05 GEMM tiles overlapped with the
                  peer-memory traffic of the collective): HcclAllGatherMatmul, HcclMatmulReduceScatter.
--impl reference  the baseline this target is measured against: HCCL itself builds only for Ascend (ACL runtime, the ccec
                  device compiler, libhcomm.so) and cannot run on this machine, so the reference arm is the same step done
                  unfused with the stock libraries on the same GPUs -- torch.distributed NCCL all-gather / reduce-scatter
                  plus torch.matmul (cuBLAS). That process never imports this package or loads its library.
Both arms share every line of the harness: the same shapes, seeds, timing loop, clock sampling and end-to-end pipeline.

Timing: after the warm-up steps the K-step loop is timed R times (CUDA events on the launching stream, barrier + synchronize
on both sides, max over ranks); `ms_per_step` is the median repeat, min / max are in `extra`. The operands of one step
(>= 186 MB per rank) exceed the 126 MB L2, so no step finds its inputs cached.
End to end (`e2e`): every step copies its activations from pinned host memory to the device, runs the step through the
public API and copies the step's whole output shard back to pinned host memory. Copies run on their own streams and are
double-buffered, so step i+1's upload and step i-1's download overlap step i's kernels; the host waits for each download.
(Each run uploads one input more than it computes: the prefetch of the step after the last.)
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))

M_TOTAL, HIDDEN, FFN = 8192, 8192, 28672
DECODE_M, DECODE_N = 128, 8192
REFERENCE_NOTE = ("10wvw01/hccl builds only for Ascend (ACL runtime, ccec device compiler, libhcomm.so; no setup.py / pyproject.toml, "
                  "pip reports it is not installable); this arm is the same-box baseline the target names instead: "
                  "torch.distributed NCCL collectives + torch.matmul (cuBLAS), unfused")


def _clock_sampler_class():
    """The clock sampler module, loaded by path so that the reference arm does not import the package (or its library)."""
    spec = importlib.util.spec_from_file_location("_bench_clocks", os.path.join(ROOT, "hccl_b200", "utils", "clocks.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ClockSampler


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "mxfp8"])
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--no-extras", action="store_true")
    args = ap.parse_args()
    ours = args.impl == "ours"
    impl_name = "ours" if ours else "reference"

    import torch

    if not torch.cuda.is_available():
        if ours:
            raise SystemExit("bench.py needs a CUDA device")
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device is visible to this process; " + REFERENCE_NOTE}))
        return
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("for --gpus > 1 launch with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    N = world
    mxfp8 = args.dtype == "mxfp8"

    comm = mc2 = gemm = None
    launch_count = lambda: 0                                    # noqa: E731
    if ours:
        sys.path.insert(0, ROOT)
        from hccl_b200._lib import lib
        from hccl_b200.comm import init_from_env
        from hccl_b200.ops import gemm, mc2
        import ctypes

        comm = init_from_env()
        _l = lib()
        _l.HcclGetKernelLaunchCount.restype = ctypes.c_uint64
        launch_count = lambda: int(_l.HcclGetKernelLaunchCount())   # noqa: E731
    ClockSampler = _clock_sampler_class()

    m_local, ffn_local = M_TOTAL // N, FFN // N
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    x_src = torch.randn(m_local, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)                # activations N(0,1)
    w_up = (torch.randn(ffn_local, HIDDEN, generator=g, device="cuda") * 0.02).to(torch.bfloat16)      # weights N(0,0.02)
    w_down = (torch.randn(HIDDEN, ffn_local, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    x_pinned = x_src.cpu().pin_memory()
    x_dev = [x_src, torch.empty_like(x_src)]
    x_dev[1].copy_(x_src)
    h = torch.empty(M_TOTAL, ffn_local, dtype=torch.bfloat16, device="cuda")
    out_dev = [torch.empty(m_local, HIDDEN, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    out_host = [torch.empty(m_local, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    x_full = partial = None
    if not ours and N > 1:
        x_full = torch.empty(M_TOTAL, HIDDEN, dtype=torch.bfloat16, device="cuda")
        partial = torch.empty(M_TOTAL, HIDDEN, dtype=torch.bfloat16, device="cuda")

    if mxfp8:
        if ours:
            from hccl_b200.ops import mxfp8 as mx

            wq_up, wq_down = mx.quantize(w_up), mx.quantize(w_down)        # weights are quantised once, outside the step

            def first_half(x, dst):
                mx.all_gather_matmul(comm, x, wq_up, out=dst)              # quantises the activations, gathers e4m3 + scales

            def second_half(src, dst):
                mx.matmul_reduce_scatter(comm, src, wq_down, out=dst)
        else:
            # per-tensor-scaled fp8 through torch._scaled_mm (cuBLASLt): the stock fp8 path of the installed torch
            one = torch.ones((), device="cuda")
            w_up8, w_down8 = w_up.to(torch.float8_e4m3fn), w_down.to(torch.float8_e4m3fn)
            x8_full = torch.empty(M_TOTAL, HIDDEN, dtype=torch.float8_e4m3fn, device="cuda") if N > 1 else None

            def first_half(x, dst):
                x8 = x.to(torch.float8_e4m3fn)
                if N > 1:
                    dist.all_gather_into_tensor(x8_full.view(torch.uint8), x8.view(torch.uint8))
                    x8 = x8_full
                torch._scaled_mm(x8, w_up8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=dst)

            def second_half(src, dst):
                s8 = src.to(torch.float8_e4m3fn)
                if N > 1:
                    torch._scaled_mm(s8, w_down8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=partial)
                    dist.reduce_scatter_tensor(dst, partial)
                else:
                    torch._scaled_mm(s8, w_down8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=dst)
    elif ours:
        def first_half(x, dst):
            mc2.all_gather_matmul(comm, x, w_up, out=dst)

        def second_half(src, dst):
            mc2.matmul_reduce_scatter(comm, src, w_down, out=dst)
    else:
        def first_half(x, dst):
            if N > 1:
                dist.all_gather_into_tensor(x_full, x)
                torch.matmul(x_full, w_up.t(), out=dst)
            else:
                torch.matmul(x, w_up.t(), out=dst)

        def second_half(src, dst):
            if N > 1:
                torch.matmul(src, w_down.t(), out=partial)
                dist.reduce_scatter_tensor(dst, partial)
            else:
                torch.matmul(src, w_down.t(), out=dst)

    def step(buf: int = 0):
        first_half(x_dev[buf], h)
        second_half(h, out_dev[buf])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        """ms per call of fn over `steps` calls: device time, max over ranks."""
        sync_all()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        sync_all()
        t = torch.tensor([s.elapsed_time(e) / steps], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    warmup = max(args.warmup, 3)
    repeats = max(args.repeats, 1)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(warmup):
        step()
    sync_all()
    sampler.mark()                                              # samples taken before the timed region are dropped
    launches_before = launch_count()
    samples = [timed(step, args.steps) for _ in range(repeats)]
    launches = launch_count() - launches_before
    clocks = sampler.stop() if rank == 0 else {}
    ms = statistics.median(samples)
    flops = 2 * 2.0 * M_TOTAL * HIDDEN * FFN
    tflops = flops / (ms * 1e-3) / 1e12

    # ---- end to end: pinned host -> device upload of the activations, the step, download of the whole output shard
    cur = torch.cuda.current_stream()
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_step = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0}
    for b in range(2):
        ev_step[b].record(cur)
        ev_down[b].record(s_down)

    def upload(i):
        b = i & 1
        s_up.wait_event(ev_step[b])                             # the step that last read x_dev[b] has finished
        with torch.cuda.stream(s_up):
            x_dev[b].copy_(x_pinned, non_blocking=True)
            ev_up[b].record(s_up)

    def e2e_step():
        i = state["i"]
        b = i & 1
        if i == 0:
            upload(0)
        cur.wait_event(ev_up[b])
        cur.wait_event(ev_down[b])                              # out_dev[b] has been downloaded
        step(b)
        ev_step[b].record(cur)
        upload(i + 1)                                           # the next step's input travels while this step computes
        s_down.wait_event(ev_step[b])
        with torch.cuda.stream(s_down):
            out_host[b].copy_(out_dev[b], non_blocking=True)
            ev_down[b].record(s_down)
        if i > 0:
            ev_down[b ^ 1].synchronize()                        # the host consumes the previous step's result
        state["i"] = i + 1

    def e2e_run(steps):
        for _ in range(steps):
            e2e_step()
        ev_down[(state["i"] - 1) & 1].synchronize()             # ... and the last one's before the clock stops
        s_down.synchronize()

    e2e_run(3)
    e2e_steps = max(3, args.steps)
    e2e_samples = []
    for _ in range(max(3, repeats // 2)):
        sync_all()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(cur)
        e2e_run(e2e_steps)
        cur.wait_stream(s_down)
        e.record(cur)
        sync_all()
        t = torch.tensor([s.elapsed_time(e) / e2e_steps], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_samples.append(t.item())
    e2e_ms = statistics.median(e2e_samples)
    e2e_tflops = flops / (e2e_ms * 1e-3) / 1e12
    result_checksum = float(out_host[0][0, :8].float().sum())   # the downloaded result is real data

    extra = {"ms_per_step_min": round(min(samples), 4), "ms_per_step_max": round(max(samples), 4), "repeats": repeats,
             "e2e_ms_min": round(min(e2e_samples), 4), "e2e_ms_max": round(max(e2e_samples), 4), "result_checksum": result_checksum}
    if not args.no_extras:
        # each half of the step alone, and the plain one-GPU GEMM of the same per-rank shape (no collective) next to it
        extra["agmm_ms"] = round(timed(lambda: first_half(x_dev[0], h), args.steps), 4)
        extra["mmrs_ms"] = round(timed(lambda: second_half(h, out_dev[0]), args.steps), 4)
        if N > 1 and not mxfp8:
            xg = torch.randn(M_TOTAL, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
            full_out = torch.empty(M_TOTAL, HIDDEN, dtype=torch.bfloat16, device="cuda")
            if ours:
                f1 = lambda: gemm.gemm_bf16(xg, w_up, out=h)                # noqa: E731
                f2 = lambda: gemm.gemm_bf16(h, w_down, out=full_out)        # noqa: E731
            else:
                f1 = lambda: torch.matmul(xg, w_up.t(), out=h)              # noqa: E731
                f2 = lambda: torch.matmul(h, w_down.t(), out=full_out)      # noqa: E731
            for f in (f1, f2):
                for _ in range(3):
                    f()
            extra["gemm_agmm_shape_ms"] = round(timed(f1, args.steps), 4)
            extra["gemm_mmrs_shape_ms"] = round(timed(f2, args.steps), 4)
            del xg, full_out
        if not mxfp8:
            # decode-shaped MatmulAllReduce (M=128, K=8192/N, N=8192)
            kd = HIDDEN // N
            a_d = torch.randn(DECODE_M, kd, generator=g, device="cuda").to(torch.bfloat16)
            w_d = (torch.randn(DECODE_N, kd, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
            o_d = torch.empty(DECODE_M, DECODE_N, dtype=torch.bfloat16, device="cuda")
            if ours:
                f = (lambda: mc2.matmul_all_reduce(comm, a_d, w_d, out=o_d))
            elif N > 1:
                f = (lambda: (torch.matmul(a_d, w_d.t(), out=o_d), dist.all_reduce(o_d)))
            else:
                f = (lambda: torch.matmul(a_d, w_d.t(), out=o_d))
            for _ in range(5):
                f()
            extra["matmul_allreduce_decode_us"] = round(timed(f, 50) * 1e3, 2)
        if N > 1:
            for nbytes in (64 << 10, 16 << 20, 256 << 20):
                buf = torch.empty(nbytes // 2, dtype=torch.bfloat16, device="cuda").normal_()
                f = (lambda: comm.all_reduce(buf)) if ours else (lambda: dist.all_reduce(buf))
                for _ in range(3):
                    f()
                t = timed(f, 20 if nbytes <= (16 << 20) else 5)
                extra[f"allreduce_bus_GBs_{nbytes}B"] = round(nbytes * 2 * (N - 1) / N / (t * 1e-3) / 1e9, 1)
                del buf
    if rank == 0:
        line = {
            "metric": "fused GEMM+collective TFLOP/s (AllGatherMatmul + MatmulReduceScatter, Llama-3-70B MLP shapes, TP=N)",
            "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": N, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.dtype,
            "data": "synthetic (activations N(0,1), weights N(0,0.02), random-init, seeded)",
            "impl": impl_name,
            "config": {"model": "Llama-3-70B MLP (hidden 8192, ffn 28672)", "global_batch": M_TOTAL, "seq_len": M_TOTAL,
                       "parallelism": f"tp{N}", "l2": "inputs larger than L2: operands (>= 186 MB per rank) exceed the 126 MB L2 every step",
                       "shapes": {"allgather_matmul": [m_local, HIDDEN, ffn_local], "matmul_reduce_scatter": [M_TOTAL, ffn_local, HIDDEN]}},
            "clocks": clocks,
            "e2e": {"value": round(e2e_tflops, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": x_pinned.numel() * 2, "d2h_bytes_per_step": out_host[0].numel() * 2,
                    "pipeline": "uploads and downloads on their own streams, double-buffered; the host waits for every download"},
            "gpu_launches": launches,
            "extra": extra,
        }
        if not ours:
            line["note"] = REFERENCE_NOTE
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
