"""Tensor-parallel linear layers whose forward AND backward are the fused matmul+collective kernels.

Megatron-style sequence parallelism: activations between the two linears of a block are sharded along the token
dimension, so the column-parallel linear is AllGather -> matmul and the row-parallel linear is matmul -> ReduceScatter;
their backward passes are the mirrored pair (the gradient of AllGather->matmul is matmul->ReduceScatter and vice versa).
HCCL itself ships only the primitives and the resource-context API for such fusions (reference: include/hccl_mc2.h:25-82;
docs/zh/architecture-brief.md:16 names DP/TP as the intended users); here each direction is ONE sm_100a kernel
(`hccl_b200.ops.mc2`).

CUDA bf16 tensors take the fused kernels. CPU tensors (communicator on the host simulation backend) take the same
algebra written with the plain collectives, which is what the CPU tests compare against a single-process reference.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import gemm as _gemm
from ..ops import mc2 as _mc2


# ---- the three fused primitives with a host path -----------------------------------------------------------------
def _fused_ok(*ts) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


_NATIVE_GEMM = True


def use_native_gemm(flag: bool) -> None:
    """False routes the non-fused matmuls (weight gradients) to torch.matmul; used by the NCCL + cuBLAS baseline arm."""
    global _NATIVE_GEMM
    _NATIVE_GEMM = flag


def _mm_nt(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a[M, K] @ w[N, K].T on the tcgen05 GEMM where its shape rules allow, torch.matmul otherwise."""
    if _NATIVE_GEMM and _fused_ok(a, w) and a.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        return _gemm.gemm_bf16(a.contiguous(), w.contiguous())
    return a @ w.t()


_NATIVE_WGRAD = False


def use_native_wgrad(flag: bool) -> None:
    """True computes weight gradients on the tcgen05 GEMM (needs explicit transposes of both operands, because that kernel
    takes K-major operands only); the default leaves this plain, collective-free GEMM with transposed operands to cuBLAS."""
    global _NATIVE_WGRAD
    _NATIVE_WGRAD = flag


def _wgrad(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """dW[N, K] = dy[M, N]^T @ x[M, K]"""
    if _NATIVE_WGRAD:
        return _mm_nt(dy.t().contiguous(), x.t().contiguous())
    return dy.t() @ x


def all_gather_matmul(comm, x_local: torch.Tensor, w: torch.Tensor, want_gathered: bool = False):
    """-> (all_gather_rows(x_local) @ w.T, gathered rows or None)"""
    m, k = x_local.shape
    if getattr(comm, "fused", True) and _fused_ok(x_local, w) and m % 128 == 0 and m <= 8192 and k % 8 == 0 and w.shape[0] % 8 == 0:
        gathered = torch.empty((m * comm.size, k), dtype=x_local.dtype, device=x_local.device) if want_gathered else None
        out = _mc2.all_gather_matmul(comm, x_local.contiguous(), w.contiguous(), gathered=gathered)
        return out, gathered
    gathered = torch.empty((m * comm.size, k), dtype=x_local.dtype, device=x_local.device)
    comm.all_gather(x_local.contiguous(), gathered)
    _sync(comm, x_local)
    return _mm_nt(gathered, w), (gathered if want_gathered else None)


def matmul_reduce_scatter(comm, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """-> reduce_scatter_rows(a @ w.T)"""
    m, k = a.shape
    n = w.shape[0]
    if getattr(comm, "fused", True) and _fused_ok(a, w) and m % (128 * comm.size) == 0 and m // comm.size <= 8192 and k % 8 == 0 and n % 8 == 0:
        return _mc2.matmul_reduce_scatter(comm, a.contiguous(), w.contiguous())
    partial = _mm_nt(a, w).contiguous()
    out = torch.empty((m // comm.size, n), dtype=a.dtype, device=a.device)
    comm.reduce_scatter(partial, out)
    _sync(comm, a)
    return out


def matmul_all_reduce(comm, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """-> all_reduce(a @ w.T)"""
    if getattr(comm, "fused", True) and _fused_ok(a, w) and a.shape[1] % 8 == 0 and w.shape[0] % 64 == 0:
        return _mc2.matmul_all_reduce(comm, a.contiguous(), w.contiguous())
    out = _mm_nt(a, w).contiguous()
    comm.all_reduce(out)
    _sync(comm, a)
    return out


def _sync(comm, ref: torch.Tensor) -> None:
    if not ref.is_cuda:
        comm.synchronize()      # host backend: operators are queued on a worker


# ---- autograd ------------------------------------------------------------------------------------------------------
class _ColumnSeqParallel(torch.autograd.Function):
    """y[R*m, Nl] = AG(x[m, K]) @ W[Nl, K]^T"""

    @staticmethod
    def forward(ctx, x_local, w, comm):
        out, gathered = all_gather_matmul(comm, x_local, w, want_gathered=True)
        ctx.comm = comm
        ctx.save_for_backward(gathered, w)
        return out

    @staticmethod
    def backward(ctx, dy):
        gathered, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = matmul_reduce_scatter(ctx.comm, dy, w.t().contiguous())          # RS(dy @ W): the mirror of the forward
        dw = _wgrad(dy, gathered)                                               # dy^T @ AG(x)
        return dx, dw, None


class _RowSeqParallel(torch.autograd.Function):
    """y[M/R, N] = RS(x[M, Kl] @ W[N, Kl]^T)"""

    @staticmethod
    def forward(ctx, x, w, comm):
        ctx.comm = comm
        ctx.save_for_backward(x, w)
        return matmul_reduce_scatter(comm, x, w)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        dx, dyg = all_gather_matmul(ctx.comm, dy_local.contiguous(), w.t().contiguous(), want_gathered=True)   # AG(dy) @ W
        dw = _wgrad(dyg, x)                                                                                    # AG(dy)^T @ x
        return dx, dw, None


class _RowAllReduce(torch.autograd.Function):
    """y[M, N] = AR(x[M, Kl] @ W[N, Kl]^T): the decode-sized variant without sequence sharding."""

    @staticmethod
    def forward(ctx, x, w, comm):
        ctx.save_for_backward(x, w)
        return matmul_all_reduce(comm, x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        return _mm_nt(dy, w.t().contiguous()), _wgrad(dy, x), None


class _ColumnReplicatedInput(torch.autograd.Function):
    """y[M, Nl] = x[M, K] @ W[Nl, K]^T with x replicated; the input gradient is all-reduced."""

    @staticmethod
    def forward(ctx, x, w, comm):
        ctx.comm = comm
        ctx.save_for_backward(x, w)
        return _mm_nt(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = matmul_all_reduce(ctx.comm, dy, w.t().contiguous())
        return dx, _wgrad(dy, x), None


# ---- modules -------------------------------------------------------------------------------------------------------
class ColumnParallelLinear(nn.Module):
    """Weight [out_features / tp, in_features]. sequence_parallel=True: input [tokens / tp, in] -> output [tokens, out / tp]."""

    def __init__(self, comm, in_features: int, out_features: int, *, sequence_parallel: bool = True, dtype=torch.bfloat16, device=None,
                 init_std: float = 0.02, seed: Optional[int] = None):
        super().__init__()
        assert out_features % comm.size == 0
        self.comm, self.sequence_parallel = comm, sequence_parallel
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features // comm.size, in_features, dtype=dtype, device=device)
        _init_shard(w, init_std, seed, comm.rank, dim=0, full=out_features)
        self.weight = nn.Parameter(w)

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        fn = _ColumnSeqParallel if self.sequence_parallel else _ColumnReplicatedInput
        y = fn.apply(x2, self.weight, self.comm)
        if self.sequence_parallel:
            return y
        return y.reshape(*lead, -1)


class RowParallelLinear(nn.Module):
    """Weight [out_features, in_features / tp]. sequence_parallel=True: input [tokens, in / tp] -> output [tokens / tp, out]."""

    def __init__(self, comm, in_features: int, out_features: int, *, sequence_parallel: bool = True, dtype=torch.bfloat16, device=None,
                 init_std: float = 0.02, seed: Optional[int] = None):
        super().__init__()
        assert in_features % comm.size == 0
        self.comm, self.sequence_parallel = comm, sequence_parallel
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features, in_features // comm.size, dtype=dtype, device=device)
        _init_shard(w, init_std, seed, comm.rank, dim=1, full=in_features)
        self.weight = nn.Parameter(w)

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features // self.comm.size)
        fn = _RowSeqParallel if self.sequence_parallel else _RowAllReduce
        y = fn.apply(x2, self.weight, self.comm)
        if self.sequence_parallel:
            return y
        return y.reshape(*lead, -1)


def _init_shard(w: torch.Tensor, std: float, seed: Optional[int], rank: int, dim: int, full: int) -> None:
    """Every rank draws the FULL matrix from the same seed and keeps its shard, so a TP model equals the unsharded one."""
    if seed is None:
        nn.init.normal_(w, std=std)
        return
    g = torch.Generator().manual_seed(seed)
    shape = list(w.shape)
    shape[dim] = full
    fullw = torch.randn(shape, generator=g, dtype=torch.float32) * std
    n = w.shape[dim]
    w.copy_(fullw.narrow(dim, rank * n, n).to(w.dtype))


class TensorParallelMLP(nn.Module):
    """SwiGLU MLP: gate/up projections column-parallel (one fused AllGather-matmul over their concatenation), down
    projection row-parallel (matmul-ReduceScatter). Input and output are token-sharded [tokens / tp, hidden]."""

    def __init__(self, comm, hidden: int, ffn: int, *, dtype=torch.bfloat16, device=None, seed: Optional[int] = None):
        super().__init__()
        self.comm = comm
        self.ffn_local = ffn // comm.size
        self.gate_up = ColumnParallelLinear(comm, hidden, 2 * ffn, dtype=dtype, device=device, seed=None)
        self.down = RowParallelLinear(comm, ffn, hidden, dtype=dtype, device=device, seed=seed + 1 if seed is not None else None,
                                      init_std=0.02 / math.sqrt(2))
        if seed is not None:   # gate and up drawn separately so that the shard layout [gate_local; up_local] matches an unsharded model
            g = torch.empty(self.ffn_local, hidden, dtype=dtype)
            u = torch.empty(self.ffn_local, hidden, dtype=dtype)
            _init_shard(g, 0.02, seed + 2, comm.rank, 0, ffn)
            _init_shard(u, 0.02, seed + 3, comm.rank, 0, ffn)
            with torch.no_grad():
                self.gate_up.weight.copy_(torch.cat([g, u]).to(self.gate_up.weight.device))

    def forward(self, x_local):
        gu = self.gate_up(x_local)
        g, u = gu[:, : self.ffn_local], gu[:, self.ffn_local:]
        return self.down(torch.nn.functional.silu(g) * u)
