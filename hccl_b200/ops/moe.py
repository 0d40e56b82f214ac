"""Expert-parallel MoE dispatch / combine (one fused kernel per direction; see include/hccl/hccl_moe.h)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .._lib import check, lib


class HcclMoeConfig(ctypes.Structure):
    _fields_ = [("numExperts", ctypes.c_uint32), ("topK", ctypes.c_uint32), ("hidden", ctypes.c_uint32), ("maxTokens", ctypes.c_uint32),
                ("maxRecvRows", ctypes.c_uint32), ("mxfp8", ctypes.c_uint32), ("reserved", ctypes.c_uint32 * 4)]


def _decl():
    l = lib()
    if not getattr(l, "_moe_declared", False):
        vp, u32, P = ctypes.c_void_p, ctypes.c_uint32, ctypes.POINTER
        l.HcclMoeCreate.argtypes = [vp, P(HcclMoeConfig), P(vp)]
        l.HcclMoeDestroy.argtypes = [vp]
        l.HcclMoeDispatch.argtypes = [vp, vp, vp, u32, P(vp), P(vp), P(vp), P(vp), vp]
        l.HcclMoeGetExpertOutBuffer.argtypes = [vp, P(vp)]
        l.HcclMoeCombine.argtypes = [vp, vp, vp, u32, vp]
        l.HcclEmuMoeRoundTrip.argtypes = [vp, P(HcclMoeConfig), P(vp), P(vp), P(vp), P(vp), u32, P(vp), u32]
        for f in (l.HcclMoeCreate, l.HcclMoeDestroy, l.HcclMoeDispatch, l.HcclMoeGetExpertOutBuffer, l.HcclMoeCombine, l.HcclEmuMoeRoundTrip):
            f.restype = ctypes.c_int
        l._moe_declared = True
    return l


def _view(ptr: int, shape, dtype, device) -> torch.Tensor:
    """Tensor aliasing `ptr` (memory owned by the communicator's symmetric heap)."""
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty((), dtype=dtype).element_size()

    class _Holder:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}

    return torch.as_tensor(_Holder(), device=device).view(dtype).view(*shape)


class MoeDispatcher:
    """Keeps the symmetric buffers of one MoE layer configuration.

    dispatch(x, topk_idx) -> (recv_x, recv_scales, recv_counts, recv_src): tensors that alias the symmetric receive buffer
    (rows grouped by local expert; use recv_counts to split). Write the expert outputs into `expert_out` (same row order)
    and call combine(topk_weights) to get the weighted sum back on the rank that owns each token.
    """

    def __init__(self, comm, num_experts: int, top_k: int, hidden: int, max_tokens: int, max_recv_rows: int = 0, mxfp8: bool = False):
        self.comm = comm
        self.cfg = HcclMoeConfig(num_experts, top_k, hidden, max_tokens, max_recv_rows, int(mxfp8))
        self.cap = max_recv_rows or 2 * max_tokens * top_k
        h = ctypes.c_void_p()
        check(_decl().HcclMoeCreate(comm.handle, ctypes.byref(self.cfg), ctypes.byref(h)), "HcclMoeCreate")
        self._h = h
        y = ctypes.c_void_p()
        check(_decl().HcclMoeGetExpertOutBuffer(self._h, ctypes.byref(y)), "HcclMoeGetExpertOutBuffer")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.expert_out = _view(y.value, (self.cap, hidden), torch.bfloat16, dev)
        self.local_experts = num_experts // comm.size
        self.mxfp8 = mxfp8
        self.hidden = hidden
        self._tokens = 0

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, stream=None) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor, torch.Tensor]:
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
        s = (torch.cuda.current_stream() if stream is None else stream).cuda_stream
        rx, rs, rc, rsrc = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        check(_decl().HcclMoeDispatch(self._h, x.data_ptr(), topk_idx.data_ptr(), x.shape[0], ctypes.byref(rx), ctypes.byref(rs), ctypes.byref(rc),
                                      ctypes.byref(rsrc), s), "HcclMoeDispatch")
        self._tokens = x.shape[0]
        dev = x.device
        recv_x = _view(rx.value, (self.cap, self.hidden), torch.float8_e4m3fn if self.mxfp8 else torch.bfloat16, dev)
        recv_scales = _view(rs.value, (self.cap, self.hidden // 32), torch.uint8, dev) if self.mxfp8 else None
        return recv_x, recv_scales, _view(rc.value, (self.local_experts,), torch.int32, dev), _view(rsrc.value, (self.cap,), torch.int32, dev)

    def combine(self, topk_weights: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        assert topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
        if out is None:
            out = torch.empty((self._tokens, self.hidden), dtype=torch.bfloat16, device=topk_weights.device)
        s = (torch.cuda.current_stream() if stream is None else stream).cuda_stream
        check(_decl().HcclMoeCombine(self._h, topk_weights.data_ptr(), out.data_ptr(), self._tokens, s), "HcclMoeCombine")
        return out

    def close(self):
        if self._h:
            _decl().HcclMoeDestroy(self._h)
            self._h = None
