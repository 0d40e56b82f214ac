"""Single-GPU emulation of a multi-rank communicator for kernel tests.

All ranks' heaps live on the current CUDA device and each operator chunk is ONE cooperative launch whose
`blockIdx.y` is the rank, so CTAs that wait for each other are guaranteed to be co-resident. This exercises the
flag protocols, index arithmetic and reductions of the SM-engine kernels without NVLink.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from .._lib import check, lib
from ..types import DataType, ReduceOp, from_torch


def _decl():
    l = lib()
    vp, u32, u64, i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int
    P = ctypes.POINTER
    l.HcclEmuCreate.argtypes = [u32, u64, u64, u32, P(vp)]
    l.HcclEmuDestroy.argtypes = [vp]
    l.HcclEmuRun.argtypes = [vp, i32, ctypes.c_char_p, P(vp), P(vp), u64, i32, i32, u32, P(u64), u32]
    l.HcclEmuBatchSendRecv.argtypes = [vp, u32, P(u32), P(u32), P(vp), P(vp), P(u64)]
    l.HcclEmuStatus.argtypes = [vp, u32, P(u32), i32]
    l.HcclEmuLonelyBarrier.argtypes = [vp, u32]
    l.HcclEmuFusedRun.argtypes = [vp, i32, P(vp), P(vp), P(vp), u64, u64, u64, u32, u32]
    l.HcclEmuFusedRun.restype = ctypes.c_int
    l.HcclEmuFusedRunMx.argtypes = [vp, i32, P(vp), P(vp), P(vp), P(vp), P(vp), u64, u64, u64, u32, u32]
    l.HcclEmuFusedRunMx.restype = ctypes.c_int
    for f in (l.HcclEmuCreate, l.HcclEmuDestroy, l.HcclEmuRun, l.HcclEmuBatchSendRecv, l.HcclEmuStatus, l.HcclEmuLonelyBarrier):
        f.restype = ctypes.c_int
    return l


class EmuWorld:
    def __init__(self, nranks: int, ccl_bytes: int = 8 << 20, wait_timeout_ms: int = 2000, arena_bytes: int = 0):
        self._l = _decl()
        self.n = nranks
        h = ctypes.c_void_p()
        check(self._l.HcclEmuCreate(nranks, ccl_bytes, arena_bytes, wait_timeout_ms, ctypes.byref(h)), "HcclEmuCreate")
        self._h = h

    def close(self):
        if self._h:
            self._l.HcclEmuDestroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _ptrs(self, tensors: Optional[Sequence[Optional[torch.Tensor]]]):
        if tensors is None:
            return None
        arr = (ctypes.c_void_p * self.n)()
        for i, t in enumerate(tensors):
            arr[i] = t.data_ptr() if t is not None else None
        return arr

    def run(self, op: int, alg: str, ins, outs, count: int, dtype: torch.dtype, reduce_op: ReduceOp = ReduceOp.SUM, root: int = 0,
            counts: Optional[Sequence[int]] = None, max_ctas: int = 4) -> int:
        cm = (ctypes.c_uint64 * len(counts))(*counts) if counts is not None else None
        rc = self._l.HcclEmuRun(self._h, op, alg.encode(), self._ptrs(ins), self._ptrs(outs), count, int(from_torch(dtype)), int(reduce_op), root,
                                cm, max_ctas)
        torch.cuda.synchronize()
        return rc

    def batch_send_recv(self, transfers: List[tuple]) -> int:
        """transfers: (src_rank, dst_rank, src_tensor, dst_tensor)"""
        n = len(transfers)
        s = (ctypes.c_uint32 * n)(*[t[0] for t in transfers])
        d = (ctypes.c_uint32 * n)(*[t[1] for t in transfers])
        sb = (ctypes.c_void_p * n)(*[t[2].data_ptr() for t in transfers])
        db = (ctypes.c_void_p * n)(*[t[3].data_ptr() for t in transfers])
        by = (ctypes.c_uint64 * n)(*[t[2].numel() * t[2].element_size() for t in transfers])
        rc = self._l.HcclEmuBatchSendRecv(self._h, n, s, d, sb, db, by)
        torch.cuda.synchronize()
        return rc

    def fused(self, kind: int, a_list, b_list, out_list, m: int, n: int, k: int, ctas_per_rank: int, comm_ctas: int = 2) -> int:
        """kind 0 AllGatherMatmul (m = rows per rank), 1 MatmulReduceScatter, 2 MatmulAllReduce"""
        rc = self._l.HcclEmuFusedRun(self._h, kind, self._ptrs(a_list), self._ptrs(b_list), self._ptrs(out_list), m, n, k, ctas_per_rank, comm_ctas)
        torch.cuda.synchronize()
        return rc

    def fused_mx(self, kind: int, a_list, b_list, out_list, m: int, n: int, k: int, ctas_per_rank: int, comm_ctas: int = 2) -> int:
        """The same operators on block-scaled fp8 operands; a_list / b_list hold `ops.mxfp8.MxTensor`s."""
        rc = self._l.HcclEmuFusedRunMx(self._h, kind, self._ptrs([t.payload for t in a_list]), self._ptrs([t.scales for t in a_list]),
                                       self._ptrs([t.payload for t in b_list]), self._ptrs([t.scales for t in b_list]), self._ptrs(out_list), m, n, k,
                                       ctas_per_rank, comm_ctas)
        torch.cuda.synchronize()
        return rc

    def arena_tensor(self, rank: int, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A tensor over `numel` elements at byte `offset` of the rank's arena: memory at the same heap offset on every emulated
        rank, i.e. what a registered window of a symmetric allocation is on a real communicator."""
        base, size = ctypes.c_void_p(), ctypes.c_uint64()
        self._l.HcclEmuArena.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint64)]
        check(self._l.HcclEmuArena(self._h, rank, ctypes.byref(base), ctypes.byref(size)), "HcclEmuArena")
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        if offset + nbytes > size.value:
            raise ValueError("arena window out of range")

        class _Window:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (base.value + offset, False), "version": 3, "strides": None}

        return torch.as_tensor(_Window(), device="cuda").view(dtype)

    def trace(self, rank: int, max_records: int = 64):
        """Device-side records of the rank's most recent kernels: dicts with seq, syncs and %globaltimer stamps in ns."""
        rows = (ctypes.c_uint64 * (6 * max_records))()
        n = ctypes.c_uint32()
        self._l.HcclEmuTrace.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint32)]
        check(self._l.HcclEmuTrace(self._h, rank, rows, max_records, ctypes.byref(n)), "HcclEmuTrace")
        keys = ("seq", "syncs", "enter", "first_sync", "last_sync", "leave")
        return [dict(zip(keys, rows[6 * i:6 * i + 6])) for i in range(n.value)]

    def status(self, rank: int, clear: bool = False):
        out = (ctypes.c_uint32 * 8)()
        check(self._l.HcclEmuStatus(self._h, rank, out, int(clear)), "HcclEmuStatus")
        return list(out)

    def lonely_barrier(self, rank: int) -> int:
        return self._l.HcclEmuLonelyBarrier(self._h, rank)
