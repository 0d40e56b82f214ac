"""Fused matmul + collective operators (one sm_100a kernel each). Weights are [N, K] (torch Linear layout)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .._lib import check, lib
from ..types import DataType


def _decl():
    l = lib()
    if not getattr(l, "_mc2_declared", False):
        vp, u64, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int
        l.HcclAllGatherMatmul.argtypes = [vp, vp, vp, vp, u64, u64, u64, i32, vp, vp]
        l.HcclMatmulReduceScatter.argtypes = [vp, vp, vp, u64, u64, u64, i32, vp, vp]
        l.HcclMatmulAllReduce.argtypes = [vp, vp, vp, u64, u64, u64, i32, vp, vp]
        for f in (l.HcclAllGatherMatmul, l.HcclMatmulReduceScatter, l.HcclMatmulAllReduce):
            f.restype = ctypes.c_int
        l._mc2_declared = True
    return l


def _stream(stream):
    return (torch.cuda.current_stream() if stream is None else stream).cuda_stream


def _chk(*ts):
    for t in ts:
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise ValueError("fused ops take contiguous bf16 CUDA tensors")


def all_gather_matmul(comm, a_local: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                      gathered: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[size*m, N] = all_gather(a_local[m, K]) @ w[N, K].T"""
    _chk(a_local, w)
    m, k = a_local.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m * comm.size, n), dtype=torch.bfloat16, device=a_local.device)
    check(_decl().HcclAllGatherMatmul(a_local.data_ptr(), w.data_ptr(), out.data_ptr(), gathered.data_ptr() if gathered is not None else None,
                                      m, n, k, int(DataType.BFP16), comm.handle, _stream(stream)), "HcclAllGatherMatmul")
    return out


def matmul_reduce_scatter(comm, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[M/size, N] = reduce_scatter_rows(a[M, Klocal] @ w[N, Klocal].T)"""
    _chk(a, w)
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m // comm.size, n), dtype=torch.bfloat16, device=a.device)
    check(_decl().HcclMatmulReduceScatter(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, int(DataType.BFP16), comm.handle, _stream(stream)),
          "HcclMatmulReduceScatter")
    return out


def matmul_all_reduce(comm, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[M, N] = all_reduce(a[M, Klocal] @ w[N, Klocal].T)"""
    _chk(a, w)
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    check(_decl().HcclMatmulAllReduce(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, int(DataType.BFP16), comm.handle, _stream(stream)),
          "HcclMatmulAllReduce")
    return out
