"""MXFP8 (block-scaled fp8) operands and the operators that consume them.

An `MxTensor` is a [rows, K] matrix stored as e4m3 elements plus one e8m0 (power-of-two) scale per 1 x 32 block of K, in
the layout the block-scaled tcgen05 kernels read directly (`include/hccl/hccl_mc2.h`, part 3). `quantize` runs the
library's CUDA quantiser; `quantize_reference` / `dequantize` are plain PyTorch restatements of the same rule, used by
the tests and as documentation of the format.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from .._lib import check, lib


@dataclass
class MxTensor:
    payload: torch.Tensor      # [rows, K] uint8 (e4m3 bit patterns)
    scales: torch.Tensor       # [ceil(rows/128) * (K/128) * 512] uint8 (e8m0), atom layout
    rows: int
    k: int


def _decl():
    l = lib()
    if not getattr(l, "_mx_declared", False):
        vp, u64, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int
        l.HcclMxfp8ScaleBytes.argtypes = [u64, u64]
        l.HcclMxfp8ScaleBytes.restype = u64
        l.HcclQuantizeMxfp8.argtypes = [vp, vp, vp, u64, u64, vp]
        l.HcclGemmMxfp8Variant.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, i32, i32, vp]
        l.HcclAllGatherMatmulMxfp8.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, vp, vp]
        l.HcclMatmulReduceScatterMxfp8.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, vp, vp]
        l.HcclMatmulAllReduceMxfp8.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, vp, vp]
        for f in (l.HcclQuantizeMxfp8, l.HcclGemmMxfp8Variant, l.HcclAllGatherMatmulMxfp8, l.HcclMatmulReduceScatterMxfp8, l.HcclMatmulAllReduceMxfp8):
            f.restype = ctypes.c_int
        l._mx_declared = True
    return l


def _stream(stream):
    return (torch.cuda.current_stream() if stream is None else stream).cuda_stream


def scale_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128) * (k // 128) * 512


def empty_like_quantized(rows: int, k: int, device) -> MxTensor:
    return MxTensor(torch.empty((rows, k), dtype=torch.uint8, device=device), torch.empty(scale_bytes(rows, k), dtype=torch.uint8, device=device), rows, k)


def quantize(x: torch.Tensor, out: Optional[MxTensor] = None, stream=None) -> MxTensor:
    """bf16 [rows, K] (K % 128 == 0) -> MxTensor, on the GPU."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 2):
        raise ValueError("quantize takes a contiguous 2-D bf16 CUDA tensor")
    rows, k = x.shape
    if out is None:
        out = empty_like_quantized(rows, k, x.device)
    check(_decl().HcclQuantizeMxfp8(x.data_ptr(), out.payload.data_ptr(), out.scales.data_ptr(), rows, k, _stream(stream)), "HcclQuantizeMxfp8")
    return out


def _scale_index(rows_padded: int, k: int, device) -> torch.Tensor:
    """Byte offset of the scale of (row r, block kb) inside the atom array, as a [rows_padded, K/32] int64 tensor."""
    r = torch.arange(rows_padded, device=device).view(-1, 1)
    kb = torch.arange(k // 32, device=device).view(1, -1)
    return ((r // 128) * (k // 128) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4


def quantize_reference(x: torch.Tensor) -> MxTensor:
    """The same quantisation rule in plain PyTorch (any device)."""
    rows, k = x.shape
    v = x.float().view(rows, k // 32, 32)
    amax = v.abs().amax(dim=2)
    e = (amax.view(torch.int32) >> 23) & 0xFF                      # biased floor(log2(amax)); 0 for zero
    se = (e - 8).clamp(0, 254)
    inv = ((254 - se) << 23).to(torch.int32).view(torch.float32)   # 2^(127 - se)
    q = (v * inv.unsqueeze(2)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).view(rows, k)
    rows_padded = (rows + 127) // 128 * 128
    se_p = torch.full((rows_padded, k // 32), 127, dtype=torch.uint8, device=x.device)
    se_p[:rows] = se.to(torch.uint8)
    scales = torch.zeros(scale_bytes(rows, k), dtype=torch.uint8, device=x.device)
    scales[_scale_index(rows_padded, k, x.device).reshape(-1)] = se_p.reshape(-1)
    return MxTensor(q.contiguous(), scales, rows, k)


def dequantize(t: MxTensor) -> torch.Tensor:
    """MxTensor -> fp32 [rows, K] (exact)."""
    rows_padded = (t.rows + 127) // 128 * 128
    se = t.scales[_scale_index(rows_padded, t.k, t.scales.device).reshape(-1)].view(rows_padded, t.k // 32)[:t.rows]
    scale = (se.to(torch.int32) << 23).view(torch.float32)        # 2^(se - 127); se = 0 reads as 0.0 (a denormal-free stand-in for 2^-127)
    scale = torch.where(se == 0, torch.full_like(scale, 2.0 ** -126) * 0.5, scale)
    v = t.payload.view(torch.float8_e4m3fn).float().view(t.rows, t.k // 32, 32)
    return (v * scale.unsqueeze(2)).view(t.rows, t.k)


# Quantised activations of the fused operators live in buffers that are reused per (shape, device, stream): work on one stream is
# ordered, so the next quantisation cannot overtake the kernel that still reads the previous one, and stable addresses let the native
# side reuse its cached tensor maps instead of encoding eight of them per call.
_ACT_BUFFERS = {}


def _as_mx_fresh(x, stream=None) -> MxTensor:
    """Second operands (weights): quantise once outside the step and pass the MxTensor; a bf16 tensor gets a buffer of its own."""
    return x if isinstance(x, MxTensor) else quantize(x, stream=stream)


def _as_mx(x, stream=None) -> MxTensor:
    if isinstance(x, MxTensor):
        return x
    key = (x.shape[0], x.shape[1], x.device, _stream(stream))
    buf = _ACT_BUFFERS.get(key)
    if buf is None:
        if len(_ACT_BUFFERS) >= 16:
            _ACT_BUFFERS.clear()
        buf = _ACT_BUFFERS[key] = empty_like_quantized(x.shape[0], x.shape[1], x.device)
    return quantize(x, out=buf, stream=stream)


def gemm(a, w, out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16, tile_n: int = 0, stream=None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T with both operands block-scaled (bf16 inputs are quantised first)."""
    a, w = _as_mx(a, stream), _as_mx_fresh(w, stream)
    assert a.k == w.k
    if out is None:
        out = torch.empty((a.rows, w.rows), dtype=out_dtype, device=a.payload.device)
    check(_decl().HcclGemmMxfp8Variant(a.payload.data_ptr(), a.scales.data_ptr(), w.payload.data_ptr(), w.scales.data_ptr(), out.data_ptr(), a.rows, w.rows,
                                       a.k, int(out.dtype == torch.float32), tile_n, _stream(stream)), "HcclGemmMxfp8")
    return out


def all_gather_matmul(comm, a_local, w, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[size*m, N] = all_gather(a_local[m, K]) @ w[N, K]^T; the gather moves e4m3 bytes and scales."""
    a, w = _as_mx(a_local, stream), _as_mx_fresh(w, stream)
    if out is None:
        out = torch.empty((a.rows * comm.size, w.rows), dtype=torch.bfloat16, device=a.payload.device)
    check(_decl().HcclAllGatherMatmulMxfp8(a.payload.data_ptr(), a.scales.data_ptr(), w.payload.data_ptr(), w.scales.data_ptr(), out.data_ptr(), a.rows, w.rows,
                                           a.k, comm.handle, _stream(stream)), "HcclAllGatherMatmulMxfp8")
    return out


def matmul_reduce_scatter(comm, a, w, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[M/size, N] = reduce_scatter_rows(a[M, Klocal] @ w[N, Klocal]^T); partials travel as bf16, summed in rank order."""
    a, w = _as_mx(a, stream), _as_mx_fresh(w, stream)
    if out is None:
        out = torch.empty((a.rows // comm.size, w.rows), dtype=torch.bfloat16, device=a.payload.device)
    check(_decl().HcclMatmulReduceScatterMxfp8(a.payload.data_ptr(), a.scales.data_ptr(), w.payload.data_ptr(), w.scales.data_ptr(), out.data_ptr(), a.rows,
                                               w.rows, a.k, comm.handle, _stream(stream)), "HcclMatmulReduceScatterMxfp8")
    return out


def matmul_all_reduce(comm, a, w, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    a, w = _as_mx(a, stream), _as_mx_fresh(w, stream)
    if out is None:
        out = torch.empty((a.rows, w.rows), dtype=torch.bfloat16, device=a.payload.device)
    check(_decl().HcclMatmulAllReduceMxfp8(a.payload.data_ptr(), a.scales.data_ptr(), w.payload.data_ptr(), w.scales.data_ptr(), out.data_ptr(), a.rows,
                                           w.rows, a.k, comm.handle, _stream(stream)), "HcclMatmulAllReduceMxfp8")
    return out
