"""tcgen05 GEMM (sm_100a): `gemm_bf16(a, w)` = a @ w.T with bf16 operands and fp32 accumulation in tensor memory."""
from __future__ import annotations

import ctypes

import torch

from .._lib import check, lib


def _decl():
    l = lib()
    if not getattr(l, "_gemm_declared", False):
        l.HcclGemmBf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                   ctypes.c_int, ctypes.c_void_p]
        l.HcclGemmBf16.restype = ctypes.c_int
        l.HcclGemmBf16Variant.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        l.HcclGemmBf16Variant.restype = ctypes.c_int
        l.HcclGemmCheckError.argtypes = []
        l.HcclGemmCheckError.restype = ctypes.c_int
        l._gemm_declared = True
    return l


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
              stream=None, variant: int = 0) -> torch.Tensor:
    """a: [M, K] bf16, w: [N, K] bf16 (both row-major) -> [M, N] in `out_dtype` (bf16 or fp32).
    variant: 0 automatic, 1 one-CTA tiles, 2 CTA-pair (cta_group::2) 256 x 256 tiles."""
    if not (a.is_cuda and w.is_cuda):
        raise RuntimeError("gemm_bf16 needs CUDA tensors (the tcgen05 kernel has no CPU path)")
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    M, K = a.shape
    N, K2 = w.shape
    assert K == K2
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    s = torch.cuda.current_stream() if stream is None else stream
    check(_decl().HcclGemmBf16Variant(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(out.dtype == torch.float32), variant, s.cuda_stream),
          "HcclGemmBf16")
    return out


def check_error() -> None:
    check(_decl().HcclGemmCheckError(), "HcclGemmCheckError")
