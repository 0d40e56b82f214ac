"""Collective primitive sweep: bus GB/s of this library against NCCL on the same GPUs.

Launch:  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
             benchmarks/coll_sweep.py [--ops allreduce,allgather,...] [--dtypes fp32,bf16] [--min-bytes 1024] [--max-bytes 1073741824]
Per-rank message sizes are powers of two; inputs are uniform[-1,1] seeded with rank*1000 + size_index. Every number is
device time (CUDA events on the launching stream, after warm-up), max over ranks. busBW = algBW * {allreduce 2(n-1)/n;
allgather / reducescatter / alltoall (n-1)/n; broadcast 1}. Results go to stdout (table) and, with --json, to a file.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from hccl_b200.comm import init_from_env  # noqa: E402

DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


HOST_US = {}


def native_host_us(comm):
    """Mean time the last 16 calls spent inside the native library (entry to return), from the communicator's op ring."""
    import ctypes

    from hccl_b200._lib import lib

    class Rec(ctypes.Structure):
        _fields_ = [("seq", ctypes.c_uint64), ("opType", ctypes.c_uint32), ("dataType", ctypes.c_uint32), ("reduceOp", ctypes.c_uint32),
                    ("root", ctypes.c_uint32), ("engine", ctypes.c_uint32), ("pad", ctypes.c_uint32), ("count", ctypes.c_uint64),
                    ("algName", ctypes.c_char * 64), ("beginNs", ctypes.c_uint64), ("endNs", ctypes.c_uint64)]
    recs = (Rec * 16)()
    n = ctypes.c_uint32()
    if lib().HcclGetLastOps(ctypes.c_void_p(comm.handle), recs, 16, ctypes.byref(n)) != 0 or n.value == 0:
        return float("nan"), ""
    return sum(recs[i].endNs - recs[i].beginNs for i in range(n.value)) / n.value / 1e3, recs[n.value - 1].algName.decode()


REPEATS = 1


def time_fn(fn, iters, warmup, tag=None):
    """Seconds per call: device time of `iters` back-to-back calls, max over ranks; the median of REPEATS such loops (a single host
    stall of a few milliseconds on any rank would otherwise decide a row)."""
    import time
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(REPEATS):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        h0 = time.perf_counter()
        for _ in range(iters):
            fn()
        h1 = time.perf_counter()            # host time to ISSUE the calls (no synchronisation inside)
        e.record()
        torch.cuda.synchronize()
        if tag is not None:
            HOST_US[tag] = (h1 - h0) / iters * 1e6
        t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        samples.append(t.item() * 1e-3)
    samples.sort()
    return samples[len(samples) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce,allgather,reducescatter,broadcast,alltoall")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--json", default="")
    ap.add_argument("--skip-nccl", action="store_true")
    ap.add_argument("--repeats", type=int, default=1, help="timed loops per row; the median is reported")
    ap.add_argument("--registered", action="store_true",
                    help="buffers of this library's calls are registered windows of the symmetric heap (zero-copy kernels from 1 MB up); "
                         "set HCCL_SYM_HEAP_MB large enough for the biggest size")
    args = ap.parse_args()
    global REPEATS
    REPEATS = max(1, args.repeats)
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))))
    comm = init_from_env()
    rank, n = comm.rank, comm.size
    rows = []
    windows = []

    def like_registered(t):
        """A registered window with t's contents (or t itself without --registered)."""
        if not args.registered:
            return t
        w = comm.sym_tensor(t.numel(), t.dtype)
        w.copy_(t)
        windows.append(w)
        return w

    for op in args.ops.split(","):
        for dname in args.dtypes.split(","):
            dtype = DT[dname]
            es = torch.empty((), dtype=dtype).element_size()
            size, idx = args.min_bytes, 0
            while size <= args.max_bytes:
                cnt = size // es
                g = torch.Generator(device="cuda").manual_seed(rank * 1000 + idx)
                iters = 200 if size <= (1 << 20) else 30 if size <= (64 << 20) else 8
                warm = 5 if size <= (64 << 20) else 3
                if op == "allreduce":
                    x = (torch.rand(cnt, generator=g, device="cuda") * 2 - 1).to(dtype)
                    y = torch.empty_like(x)
                    xo, yo = like_registered(x), like_registered(y)
                    ours = lambda: comm.all_reduce(xo, yo)
                    ref = lambda: dist.all_reduce(y)
                    factor = 2 * (n - 1) / n
                elif op == "allgather":
                    x = (torch.rand(cnt, generator=g, device="cuda") * 2 - 1).to(dtype)
                    y = torch.empty(cnt * n, dtype=dtype, device="cuda")
                    yo = like_registered(y)
                    ours = lambda: comm.all_gather(x, yo)
                    ref = lambda: dist.all_gather_into_tensor(y, x)
                    factor = (n - 1) / n * n   # size counts the per-rank message; bytes received = size * (n-1)
                elif op == "reducescatter":
                    x = (torch.rand(cnt * n, generator=g, device="cuda") * 2 - 1).to(dtype)
                    y = torch.empty(cnt, dtype=dtype, device="cuda")
                    xo = like_registered(x)
                    ours = lambda: comm.reduce_scatter(xo, y)
                    ref = lambda: dist.reduce_scatter_tensor(y, x)
                    factor = (n - 1) / n * n
                elif op == "broadcast":
                    x = (torch.rand(cnt, generator=g, device="cuda") * 2 - 1).to(dtype)
                    xo = like_registered(x)
                    ours = lambda: comm.broadcast(xo, 0)
                    ref = lambda: dist.broadcast(x, 0)
                    factor = 1.0
                elif op == "alltoall":
                    per = max(1, cnt // n)
                    x = (torch.rand(per * n, generator=g, device="cuda") * 2 - 1).to(dtype)
                    y = torch.empty_like(x)
                    ours = lambda: comm.all_to_all(x, y)
                    ref = lambda: dist.all_to_all_single(y, x)
                    factor = (n - 1) / n
                else:
                    raise SystemExit(f"unknown op {op}")
                t_ours = time_fn(ours, iters, warm, tag="ours")
                nat_us, alg_used = native_host_us(comm)
                t_ref = float("nan") if args.skip_nccl else time_fn(ref, iters, warm)
                bus_ours = size * factor / t_ours / 1e9
                bus_ref = size * factor / t_ref / 1e9
                rows.append(dict(op=op, dtype=dname, bytes=size, ranks=n, ours_us=t_ours * 1e6, nccl_us=t_ref * 1e6, ours_busGBs=bus_ours,
                                 nccl_busGBs=bus_ref, ratio=bus_ours / bus_ref if bus_ref == bus_ref else None, ours_host_issue_us=HOST_US.get("ours"), ours_native_us=nat_us, alg=alg_used))
                if rank == 0:
                    print(f"{op:13s} {dname:5s} {size:>11d} B  ours {t_ours*1e6:9.1f} us {bus_ours:8.1f} GB/s | nccl {t_ref*1e6:9.1f} us {bus_ref:8.1f} GB/s"
                          f" | x{bus_ours / bus_ref if bus_ref == bus_ref else float('nan'):.2f} | host {HOST_US.get('ours', 0):.1f} us (native {nat_us:.1f}) {alg_used}", flush=True)
                del x
                while windows:
                    comm.sym_free(windows.pop())          # reverse order of allocation, the same on every rank
                size *= 4 if size >= (1 << 22) and args.max_bytes > (1 << 28) else 2
                idx += 1
    if rank == 0 and args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    torch.cuda.synchronize()
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
