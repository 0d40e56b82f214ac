"""Llama-3-architecture decoder (RMSNorm, rotary embeddings, grouped-query attention, SwiGLU) with tensor + sequence
parallelism over a `Communicator`.

Between blocks the residual stream is sharded along the token dimension ([tokens / tp, hidden]); every linear is one of
the fused matmul+collective kernels (`hccl_b200.parallel.tensor_parallel`): QKV and gate/up are AllGather->matmul, the
attention output and down projections are matmul->ReduceScatter, the LM head is AllGather->matmul over a vocabulary
shard followed by a vocabulary-parallel cross entropy (two small all-reduces). With tp == 1 the same module is an
ordinary single-GPU decoder. The reference library has no model code: this module exists for the end-to-end
benchmarks that exercise the TP / DP paths the communication library is written for.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    ffn: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    max_seq: int = 8192

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny(vocab=512, hidden=256, layers=2, heads=8, kv_heads=4, ffn=512) -> "LlamaConfig":
        return LlamaConfig(vocab, hidden, layers, heads, kv_heads, ffn, max_seq=512)

    def param_count(self) -> int:
        hd = self.hidden // self.heads
        per_layer = self.hidden * (self.heads + 2 * self.kv_heads) * hd + self.hidden * self.hidden + 3 * self.hidden * self.ffn + 2 * self.hidden
        return self.layers * per_layer + 2 * self.vocab_size * self.hidden + self.hidden

    def flops_per_token(self, seq: int) -> float:
        """Forward + backward matmul FLOPs per token (6 x parameters in the linears + attention scores)."""
        hd = self.hidden // self.heads
        lin = self.layers * (self.hidden * (self.heads + 2 * self.kv_heads) * hd + self.hidden * self.hidden + 3 * self.hidden * self.ffn) \
            + self.vocab_size * self.hidden
        attn = self.layers * 2 * seq * self.hidden          # QK^T and PV, causal halves it, fwd only
        return 6.0 * lin + 6.0 * attn


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype, device):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.weight.replicated_under_sequence_parallel = True

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


def _rope_tables(seq: int, head_dim: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def _apply_rope(x, cos, sin):
    # x: [B, S, H, D]; rotate pairs (even, odd) halves in the "rotate_half" convention
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig, comm, dtype, device, seed):
        super().__init__()
        tp = comm.size
        assert cfg.heads % tp == 0 and cfg.kv_heads % tp == 0, "heads and kv_heads must divide by the tensor-parallel size"
        self.hd = cfg.hidden // cfg.heads
        self.h_local, self.kv_local = cfg.heads // tp, cfg.kv_heads // tp
        self.cfg = cfg
        # one column-parallel weight holding this rank's [q heads; k heads; v heads]
        self.qkv = ColumnParallelLinear(comm, cfg.hidden, (cfg.heads + 2 * cfg.kv_heads) * self.hd, dtype=dtype, device=device, seed=None)
        self.out = RowParallelLinear(comm, cfg.heads * self.hd, cfg.hidden, dtype=dtype, device=device, seed=seed + 1 if seed is not None else None,
                                     init_std=0.02 / math.sqrt(2 * cfg.layers))
        if seed is not None:
            from ..parallel.tensor_parallel import _init_shard
            parts = []
            for i, (nh, nl) in enumerate(((cfg.heads, self.h_local), (cfg.kv_heads, self.kv_local), (cfg.kv_heads, self.kv_local))):
                w = torch.empty(nl * self.hd, cfg.hidden, dtype=dtype)
                _init_shard(w, 0.02, seed + 2 + i, comm.rank, 0, nh * self.hd)
                parts.append(w)
            with torch.no_grad():
                self.qkv.weight.copy_(torch.cat(parts).to(self.qkv.weight.device))

    def forward(self, x_local, batch: int, seq: int, cos, sin):
        qkv = self.qkv(x_local)                                            # [B*S, (hl + 2 kvl) * hd]
        q, k, v = qkv.split([self.h_local * self.hd, self.kv_local * self.hd, self.kv_local * self.hd], dim=-1)
        q = _apply_rope(q.reshape(batch, seq, self.h_local, self.hd), cos, sin).transpose(1, 2)
        k = _apply_rope(k.reshape(batch, seq, self.kv_local, self.hd), cos, sin).transpose(1, 2)
        v = v.reshape(batch, seq, self.kv_local, self.hd).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.h_local != self.kv_local)
        o = o.transpose(1, 2).reshape(batch * seq, self.h_local * self.hd)
        return self.out(o)                                                  # [B*S / tp, hidden]


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig, comm, dtype, device, seed):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden, cfg.norm_eps, dtype, device)
        self.attn = Attention(cfg, comm, dtype, device, seed)
        self.mlp_norm = RMSNorm(cfg.hidden, cfg.norm_eps, dtype, device)
        self.mlp = TensorParallelMLP(comm, cfg.hidden, cfg.ffn, dtype=dtype, device=device, seed=seed + 10 if seed is not None else None)

    def forward(self, x_local, batch, seq, cos, sin):
        x_local = x_local + self.attn(self.attn_norm(x_local), batch, seq, cos, sin)
        return x_local + self.mlp(self.mlp_norm(x_local))


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Mean cross entropy over logits sharded along the vocabulary: max and sum-exp are all-reduced, the target logit is
    contributed by the rank that owns it."""

    @staticmethod
    def forward(ctx, logits_local, targets, comm, vocab_start):
        from ..types import ReduceOp
        lf = logits_local.float()
        mx = lf.max(dim=-1).values.contiguous()
        if comm.size > 1:
            comm.all_reduce(mx, op=ReduceOp.MAX)
            _sync(comm, mx)
        ex = (lf - mx[:, None]).exp()
        vloc = logits_local.shape[-1]
        mine = (targets >= vocab_start) & (targets < vocab_start + vloc)
        idx = (targets - vocab_start).clamp(0, vloc - 1)
        tgt = torch.where(mine, lf.gather(1, idx[:, None])[:, 0] - mx, torch.zeros_like(mx))
        packed = torch.stack([ex.sum(-1), tgt]).contiguous()
        if comm.size > 1:
            comm.all_reduce(packed)
            _sync(comm, packed)
        denom, tgt = packed[0], packed[1]
        loss = (denom.log() - tgt).mean()
        ctx.save_for_backward(ex / denom[:, None], mine, idx)
        return loss

    @staticmethod
    def backward(ctx, g):
        p, mine, idx = ctx.saved_tensors
        grad = p.clone()
        grad[torch.arange(p.shape[0], device=p.device)[mine], idx[mine]] -= 1.0
        return (grad * (g / p.shape[0])).to(torch.bfloat16 if p.is_cuda else torch.float32), None, None, None


def _sync(comm, t):
    if not t.is_cuda:
        comm.synchronize()


class Llama(nn.Module):
    """`forward(tokens[B, S], targets[B, S]) -> mean next-token loss` (targets given) or vocabulary-sharded logits."""

    def __init__(self, cfg: LlamaConfig, comm, *, dtype=torch.bfloat16, device=None, seed: Optional[int] = 1234):
        super().__init__()
        self.cfg, self.comm = cfg, comm
        tp = comm.size
        assert cfg.vocab_size % tp == 0
        emb = torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device)
        if seed is not None:
            emb.copy_((torch.randn(cfg.vocab_size, cfg.hidden, generator=torch.Generator().manual_seed(seed)) * 0.02).to(dtype))
        else:
            nn.init.normal_(emb, std=0.02)
        self.embed = nn.Parameter(emb)
        self.embed.replicated_under_sequence_parallel = True
        self.blocks = nn.ModuleList([Block(cfg, comm, dtype, device, seed + 100 * (i + 1) if seed is not None else None) for i in range(cfg.layers)])
        self.norm = RMSNorm(cfg.hidden, cfg.norm_eps, dtype, device)
        self.lm_head = ColumnParallelLinear(comm, cfg.hidden, cfg.vocab_size, dtype=dtype, device=device, seed=seed + 7 if seed is not None else None)
        self._rope = None

    def forward(self, tokens, targets=None):
        B, S = tokens.shape
        tp, rank = self.comm.size, self.comm.rank
        T = B * S
        assert T % tp == 0
        flat = tokens.reshape(-1)
        x = self.embed[flat[rank * (T // tp):(rank + 1) * (T // tp)]]      # this rank's token shard
        if self._rope is None or self._rope[0].shape[0] != S or self._rope[0].device != x.device:
            self._rope = _rope_tables(S, self.cfg.hidden // self.cfg.heads, self.cfg.rope_theta, x.device)
        cos, sin = self._rope
        for blk in self.blocks:
            x = blk(x, B, S, cos, sin)
        logits = self.lm_head(self.norm(x))                                # [T, vocab / tp]
        if targets is None:
            return logits
        vloc = self.cfg.vocab_size // tp
        return _VocabParallelCrossEntropy.apply(logits, targets.reshape(-1), self.comm, rank * vloc)

    def sync_replicated_grads(self) -> None:
        """Parameters replicated across the tensor-parallel group (embedding, norm scales) see only this rank's tokens:
        their gradients are summed over the group. One flattened all-reduce."""
        if self.comm.size == 1:
            return
        ps = [p for p in self.parameters() if getattr(p, "replicated_under_sequence_parallel", False) and p.grad is not None]
        if not ps:
            return
        flat = torch.cat([p.grad.reshape(-1).float() for p in ps]).contiguous()
        self.comm.all_reduce(flat)
        _sync(self.comm, flat)
        off = 0
        for p in ps:
            n = p.grad.numel()
            p.grad.copy_(flat[off:off + n].reshape(p.grad.shape).to(p.grad.dtype))
            off += n
