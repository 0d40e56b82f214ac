"""Data parallelism: bucketed gradient all-reduce overlapped with the backward pass.

Gradients are packed into flat buckets in reverse parameter order (the order in which backward produces them); when the
last gradient of a bucket arrives, the bucket is all-reduced on a communication stream while backward keeps running on
the compute stream, and `finish()` scales by 1/world, waits for the stream and scatters the results back. Through
NVSwitch every GPU reaches every peer at full bandwidth and the two-shot / NVLS all-reduce kernels are bandwidth-bound
from a few megabytes on, so buckets are sized for launch latency and overlap (default 32 MB), not for link count.

The same mechanics are available through PyTorch's own DDP by initialising torch.distributed with backend "hccl"
(`hccl_b200.parallel.process_group`); this class is the dependency-free path used with a bare `Communicator`
(reference: HCCL offers only the AllReduce primitive for this, docs/zh/architecture-brief.md:16).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn


class _Bucket:
    def __init__(self, params: List[nn.Parameter], dtype, device, comm=None):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        if comm is not None:                                 # a registered window of the symmetric heap: reduced in place by the
            self.flat = comm.sym_tensor(self.numel, dtype)   # zero-copy kernels, no staging through the scratch buffer
            self.flat.zero_()
        else:
            self.flat = torch.zeros(self.numel, dtype=dtype, device=device)
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += p.numel()
        self.pending = len(params)
        self.event: Optional[torch.cuda.Event] = None


class DataParallel:
    """Wrap a module's parameters: `dp = DataParallel(model, comm)`; after `loss.backward()` call `dp.finish()`."""

    def __init__(self, module: nn.Module, comm, *, bucket_mb: float = 32.0, grad_dtype: Optional[torch.dtype] = None, average: bool = True,
                 registered: Optional[bool] = None, grad_as_bucket_view: bool = True, max_ctas: Optional[int] = 16):
        """`max_ctas`: cap on the grid of this communicator's collective kernels while they overlap the backward pass (CUDA only).
        `registered`: keep the buckets in registered windows of the communicator's symmetric heap (default: on CUDA with more
        than one rank). Every rank builds the same buckets in the same order, which is what symmetric allocation asks for."""
        self.comm, self.average = comm, average
        # The all-reduce shares the GPU with the backward pass: with the kernels' own grid (64-96 CTAs for a 32 MB bucket) a
        # Llama-3-8B step on 4 GPUs took 373.6 ms, capped at 32 CTAs 364.3 ms, at 16 CTAs 360.9 ms (NCCL DDP: 360.8 ms).
        # None leaves the communicator as it is.
        if max_ctas is not None and hasattr(comm, "set_max_ctas") and getattr(comm, "is_cuda", False) and comm.size > 1:
            comm.set_max_ctas(max_ctas)
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        self.device = params[0].device
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        dtype = grad_dtype or params[0].dtype
        cap = int(bucket_mb * (1 << 20)) // torch.empty(0, dtype=dtype).element_size()
        self.registered = (self.cuda and comm.size > 1) if registered is None else bool(registered)
        win = comm if self.registered else None
        self.buckets: List[_Bucket] = []
        cur, cur_n = [], 0
        for p in reversed(params):
            if cur and cur_n + p.numel() > cap:
                self.buckets.append(_Bucket(cur, dtype, self.device, win))
                cur, cur_n = [], 0
            cur.append(p)
            cur_n += p.numel()
        if cur:
            self.buckets.append(_Bucket(cur, dtype, self.device, win))
        self._where = {}
        for b in self.buckets:
            for i, p in enumerate(b.params):
                self._where[p] = (b, i)
                p.register_post_accumulate_grad_hook(self._on_grad)
                if grad_as_bucket_view and p.dtype == dtype:
                    # autograd accumulates straight into the bucket (keep the views: zero_grad(set_to_none=False)); a gradient that
                    # turns up elsewhere (set_to_none, another dtype) is copied in and out as without this option
                    p.grad = b.flat[b.offsets[i]:b.offsets[i] + p.numel()].view(p.shape)
        self.launched = 0

    def _on_grad(self, p: nn.Parameter) -> None:
        b, i = self._where[p]
        off = b.offsets[i]
        if p.grad.data_ptr() != b.flat.data_ptr() + off * b.flat.element_size():
            b.flat[off:off + p.numel()].copy_(p.grad.reshape(-1))
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    def _launch(self, b: _Bucket) -> None:
        self.launched += 1
        if self.comm.size == 1:
            return
        if self.cuda:
            ready = torch.cuda.Event()
            ready.record()                                   # the bucket's last copy on the compute stream
            self.stream.wait_event(ready)
            self.comm.all_reduce(b.flat, stream=self.stream)
            b.event = torch.cuda.Event()
            b.event.record(self.stream)
        else:
            self.comm.all_reduce(b.flat)

    def finish(self) -> None:
        """Waits for every bucket, averages, and writes the reduced gradients back into `.grad`."""
        for b in self.buckets:
            if b.pending != 0:           # a parameter without gradient this step (unused branch): reduce what there is
                self._launch(b)
        if not self.cuda:
            self.comm.synchronize()
        for b in self.buckets:
            if b.event is not None:
                torch.cuda.current_stream().wait_event(b.event)
                b.event = None
            if self.average and self.comm.size > 1:
                b.flat.div_(self.comm.size)
            for p, off in zip(b.params, b.offsets):
                if p.grad is not None and p.grad.data_ptr() != b.flat.data_ptr() + off * b.flat.element_size():
                    p.grad.copy_(b.flat[off:off + p.numel()].reshape(p.grad.shape))
            b.pending = len(b.params)

    def close(self) -> None:
        """Returns registered buckets to the heap (reverse order of allocation; call it on every rank, before the communicator
        is destroyed). Buckets in ordinary device memory need no call."""
        if self.registered:
            for b in reversed(self.buckets):
                lo, hi = b.flat.data_ptr(), b.flat.data_ptr() + b.numel * b.flat.element_size()
                for p in b.params:                           # gradients that are views of the bucket would dangle
                    if p.grad is not None and lo <= p.grad.data_ptr() < hi:
                        p.grad = None
                self.comm.sym_free(b.flat)
            self.registered = False
