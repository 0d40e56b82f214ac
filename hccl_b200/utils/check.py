"""Command-line front end of the schedule checker.

    python -m hccl_b200.utils.check --op allreduce --ranks 8 --count 1000000                    # what the selector picks on the host engine
    python -m hccl_b200.utils.check --op allreduce --ranks 8 --count 1000000 --all             # every registered algorithm of the operator
    python -m hccl_b200.utils.check --op broadcast --topo 1x2x4 --root 5 --count 70001 --alg InsBroadcastSequenceMesh1DMesh1D
    python -m hccl_b200.utils.check --op alltoallv --ranks 4 --matrix 1,0,7,3,300,1,0,2,4,5,6,0,9,9,9,9
    python -m hccl_b200.utils.check --plan schedule.txt                                         # a schedule written as text
    python -m hccl_b200.utils.check --slices --op allgather --levels 8@770,4@50 --bytes 67108864   # the slice planner's cut for two levels

The checker generates every rank's schedule for the pretended topology and examines it without running it: deadlock, notifies
nobody waits for, scratch / mailbox / user-buffer bounds, unordered accesses to the same bytes, and the operator's symbolic
result. Needs no GPU. Exit status 0 when everything checked is fine, 1 otherwise.
(The reference keeps its counterpart, the verifier of generated task queues, inside its test tree:
test/st/algorithm/utils/src/hccl_verifier/checker.cc.)
"""
from __future__ import annotations

import argparse
import ctypes
import sys

from hccl_b200._lib import lib
from hccl_b200.types import DataType

OPS = {"broadcast": 1, "allreduce": 2, "reduce": 3, "send": 4, "recv": 5, "allgather": 6, "reducescatter": 7, "alltoallv": 8, "alltoallvc": 9,
       "alltoall": 10, "scatter": 12, "batchsendrecv": 13, "barrier": 14, "allgatherv": 15, "reducescatterv": 16}
DTYPES = {"int8": DataType.INT8, "int32": DataType.INT32, "fp16": DataType.FP16, "fp32": DataType.FP32, "bf16": DataType.BFP16,
          "int64": DataType.INT64, "fp64": DataType.FP64}


def algorithms(op: int) -> list[str]:
    buf = ctypes.create_string_buffer(1 << 14)
    if lib().HcclListAlgorithms(op, buf, len(buf)) != 0:
        return []
    return [n for n in buf.value.decode().split(";") if n]


def check_algorithm(op: int, alg: str | None, topo: tuple[int, int, int], count: int, dtype: int = DataType.FP32, root: int = 0,
                    matrix: list[int] | None = None, ccl_bytes: int = 0) -> tuple[int, str]:
    """(result code, message) of HcclCheckAlgorithm; alg None = what the selector would pick on that topology."""
    l = lib()
    l.HcclCheckAlgorithm.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int,
                                     ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
    msg = ctypes.create_string_buffer(4096)
    cm = (ctypes.c_uint64 * len(matrix))(*matrix) if matrix else None
    rc = l.HcclCheckAlgorithm(op, alg.encode() if alg else None, topo[0], topo[1], topo[2], count, int(dtype), root, cm, ccl_bytes, msg, len(msg))
    return rc, msg.value.decode()


def check_plan_text(text: str) -> tuple[int, str]:
    msg = ctypes.create_string_buffer(4096)
    rc = lib().HcclCheckPlanText(text.encode(), msg, len(msg))
    return rc, msg.value.decode()


def plan_slices(op: int, level0: tuple[int, float], level1: tuple[int, float], nbytes: int) -> dict:
    """The slice planner's cut of `nbytes` per rank over two levels given as (ranks, GB/s)."""
    l = lib()
    l.HcclPlanParallelSlices.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_double, ctypes.c_uint32, ctypes.c_double, ctypes.c_uint64,
                                         ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_double),
                                         ctypes.POINTER(ctypes.c_double)]
    sb, ss = (ctypes.c_uint64 * 2)(), (ctypes.c_uint32 * 2)()
    seq, par = ctypes.c_double(), ctypes.c_double()
    rc = l.HcclPlanParallelSlices(op, level0[0], level0[1], level1[0], level1[1], nbytes, sb, ss, ctypes.byref(seq), ctypes.byref(par))
    return {"rc": rc, "share_bytes": list(sb), "share_steps": list(ss), "sequence_us": seq.value, "parallel_us": par.value}


def _topo(a) -> tuple[int, int, int]:
    if a.topo:
        parts = [int(v) for v in a.topo.lower().split("x")]
        if len(parts) != 3 or min(parts) < 1:
            raise SystemExit("--topo takes <super pods>x<servers per pod>x<ranks per server>")
        return parts[0], parts[1], parts[2]
    return 1, 1, a.ranks


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m hccl_b200.utils.check", description="schedule checker (no GPU needed)")
    ap.add_argument("--op", choices=sorted(OPS))
    ap.add_argument("--alg", help="algorithm name (default: the selector's choice on the host engine)")
    ap.add_argument("--all", action="store_true", help="every registered algorithm of the operator that fits the topology")
    ap.add_argument("--ranks", type=int, default=8, help="ranks on one server (ignored with --topo)")
    ap.add_argument("--topo", help="<super pods>x<servers per pod>x<ranks per server>")
    ap.add_argument("--count", type=int, default=4096, help="elements (per rank for gather / scatter forms)")
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="fp32")
    ap.add_argument("--root", type=int, default=0)
    ap.add_argument("--ccl-mb", type=float, default=0, help="scratch per half in MB (0 = the library's default)")
    ap.add_argument("--matrix", help="comma list: n x n send counts (alltoallv / alltoallvc) or n counts (allgatherv / reducescatterv)")
    ap.add_argument("--plan", help="file with a schedule written as text")
    ap.add_argument("--slices", action="store_true", help="print the slice planner's cut instead of checking (needs --levels and --bytes)")
    ap.add_argument("--levels", help="<ranks>@<GB/s>,<ranks>@<GB/s> for --slices")
    ap.add_argument("--bytes", type=int, default=0)
    a = ap.parse_args(argv)

    if a.plan:
        rc, msg = check_plan_text(open(a.plan).read())
        print(("ok: " if rc == 0 else "FAILED: ") + msg)
        return 0 if rc == 0 else 1
    if not a.op:
        ap.error("--op is required (or --plan)")
    op = OPS[a.op]
    if a.slices:
        if not a.levels or not a.bytes:
            ap.error("--slices needs --levels and --bytes")
        lv = [(int(p.split("@")[0]), float(p.split("@")[1])) for p in a.levels.split(",")]
        r = plan_slices(op, lv[0], lv[1], a.bytes)
        if r["rc"] != 0:
            print("the slice planner serves allgather, reducescatter and allreduce on two levels")
            return 1
        print(f"share starting inside the server: {r['share_bytes'][0]} bytes in {r['share_steps'][0]} steps; "
              f"share starting between the servers: {r['share_bytes'][1]} bytes in {r['share_steps'][1]} steps")
        print(f"modelled time: sequence {r['sequence_us']:.1f} us, parallel {r['parallel_us']:.1f} us")
        return 0
    topo = _topo(a)
    matrix = [int(v) for v in a.matrix.split(",")] if a.matrix else None
    ccl = int(a.ccl_mb * (1 << 20))
    names = algorithms(op) if a.all else [a.alg]
    if a.all:
        lib().HcclSetLogLevel(5)                  # algorithms that do not apply to the topology are reported below, not as error lines
    bad = 0
    for name in names:
        rc, msg = check_algorithm(op, name, topo, a.count, DTYPES[a.dtype], a.root, matrix, ccl)
        if a.all and rc == 5:                     # not supported: a multi-level form on one server, a count the switch path cannot align, ...
            print(f"skipped: {name} does not serve this call (layout {topo[0]}x{topo[1]}x{topo[2]}, count {a.count})")
            continue
        print(("ok: " if rc == 0 else f"FAILED ({rc}): ") + (msg or str(name)))
        bad += rc != 0
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
