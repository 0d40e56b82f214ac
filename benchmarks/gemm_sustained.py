"""Back-to-back GEMM timing under the board's power cap, with the clocks sampled while it runs.

    python benchmarks/gemm_sustained.py [--impl ours|cublas] [--variant 0|1|2] [--seconds 1.5] [--shapes MxNxK,MxNxK]

A single GEMM timed in isolation finishes before the power controller reacts; a training or serving step does not. This
runs the given shapes (default: the two GEMMs of the single-GPU headline step) in a loop for `--seconds`, times the loop with
CUDA events and reports ms per pass, TFLOP/s, and the median SM clock and power draw over the loop. One JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "cublas"])
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--seconds", type=float, default=1.5)
    ap.add_argument("--shapes", default="8192x28672x8192,8192x8192x28672")
    ap.add_argument("--tag", default="")
    a = ap.parse_args()
    shapes = [tuple(int(v) for v in s.split("x")) for s in a.shapes.split(",")]
    ops = []
    for (m, n, k) in shapes:
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        o = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        ops.append((x, w, o))
    if a.impl == "ours":
        from hccl_b200.ops import gemm

        def one_pass():
            for x, w, o in ops:
                gemm.gemm_bf16(x, w, out=o, variant=a.variant)
    else:
        def one_pass():
            for x, w, o in ops:
                torch.matmul(x, w.t(), out=o)
    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    rows = []
    stop = threading.Event()

    def sample():
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
            while not stop.is_set():
                rows.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetPowerUsage(h) / 1000.0))
                time.sleep(0.005)
        except Exception:       # noqa: BLE001 - no NVML: report times only
            pass

    # estimate passes for the requested duration
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(); one_pass(); e.record(); torch.cuda.synchronize()
    passes = max(5, int(a.seconds * 1e3 / s.elapsed_time(e)))
    th = threading.Thread(target=sample, daemon=True)
    th.start()
    time.sleep(0.05)
    skip = len(rows)
    s.record()
    for _ in range(passes):
        one_pass()
    e.record()
    torch.cuda.synchronize()
    stop.set()
    th.join(1)
    ms = s.elapsed_time(e) / passes
    flops = sum(2.0 * m * n * k for m, n, k in shapes)
    rows = rows[skip + len(rows[skip:]) // 4:]      # drop the ramp at the start of the loop
    print(json.dumps({"case": "gemm-sustained", "impl": a.impl, "variant": a.variant, "tag": a.tag, "group_m": os.environ.get("HCCL_GEMM_GROUP_M"),
                      "shapes": a.shapes, "passes": passes, "ms_per_pass": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                      "sm_mhz_median": statistics.median(r[0] for r in rows) if rows else None,
                      "power_w_median": round(statistics.median(r[1] for r in rows), 1) if rows else None,
                      "flop_per_clk_per_sm": round(flops / (ms * 1e-3) / (statistics.median(r[0] for r in rows) * 1e6) / 148, 1) if rows else None}), flush=True)


if __name__ == "__main__":
    main()
