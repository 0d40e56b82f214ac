"""Tensor + sequence parallel layers and the Llama decoder on the host simulation backend (fp32): a TP=2/4 model must
reproduce the loss and the gradients of the same model on one rank."""
import numpy as np
import pytest
import torch

from hccl_b200.models.llama import Llama, LlamaConfig
from hccl_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP
from hccl_b200.utils.sim import run_ranks


def _single(fn):
    return run_ranks(1, lambda comm, rank: fn(comm))[0]


@pytest.mark.parametrize("tp", [2, 4])
def test_mlp_matches_unsharded(tp):
    torch.manual_seed(0)
    tokens, hidden, ffn = 32, 64, 128
    x = torch.randn(tokens, hidden)
    dy = torch.randn(tokens, hidden)

    def run(comm):
        mlp = TensorParallelMLP(comm, hidden, ffn, dtype=torch.float32, seed=5)
        n = tokens // comm.size
        xl = x[comm.rank * n:(comm.rank + 1) * n].clone().requires_grad_(True)
        y = mlp(xl)
        y.backward(dy[comm.rank * n:(comm.rank + 1) * n])
        return y.detach(), xl.grad, mlp.gate_up.weight.grad, mlp.down.weight.grad

    y1, dx1, dgu1, dd1 = _single(run)
    res = run_ranks(tp, lambda comm, rank: run(comm))
    n, fl = tokens // tp, ffn // tp
    for r, (y, dx, dgu, dd) in enumerate(res):
        assert torch.allclose(y, y1[r * n:(r + 1) * n], atol=1e-5)
        assert torch.allclose(dx, dx1[r * n:(r + 1) * n], atol=1e-5)
        want_gu = torch.cat([dgu1[r * fl:(r + 1) * fl], dgu1[ffn + r * fl: ffn + (r + 1) * fl]])
        assert torch.allclose(dgu, want_gu, atol=1e-4)
        assert torch.allclose(dd, dd1[:, r * fl:(r + 1) * fl], atol=1e-4)


def test_linears_without_sequence_parallel():
    torch.manual_seed(1)
    x = torch.randn(6, 32)

    def run(comm):
        col = ColumnParallelLinear(comm, 32, 48, sequence_parallel=False, dtype=torch.float32, seed=3)
        row = RowParallelLinear(comm, 48, 16, sequence_parallel=False, dtype=torch.float32, seed=4)
        xi = x.clone().requires_grad_(True)
        y = row(torch.tanh(col(xi)))
        y.sum().backward()
        return y.detach(), xi.grad

    y1, g1 = _single(run)
    for y, g in run_ranks(2, lambda comm, rank: run(comm)):
        assert torch.allclose(y, y1, atol=1e-5) and torch.allclose(g, g1, atol=1e-5)


@pytest.mark.parametrize("tp", [2, 4])
def test_llama_loss_and_grads_match_single_rank(tp):
    cfg = LlamaConfig.tiny(vocab=64, hidden=64, layers=2, heads=8, kv_heads=4, ffn=96)
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
    targets = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)

    def run(comm):
        model = Llama(cfg, comm, dtype=torch.float32, seed=42)
        loss = model(tokens, targets)
        loss.backward()
        model.sync_replicated_grads()
        return loss.item(), model.embed.grad.clone(), model.blocks[0].attn.out.weight.grad.clone(), model.norm.weight.grad.clone(), \
            model.lm_head.weight.grad.clone()

    l1, e1, o1, n1, h1 = _single(run)
    assert abs(l1 - np.log(cfg.vocab_size)) < 0.5          # random init: loss near ln(V)
    res = run_ranks(tp, lambda comm, rank: run(comm))
    kl = cfg.hidden // tp
    vl = cfg.vocab_size // tp
    for r, (l, e, o, n, h) in enumerate(res):
        assert abs(l - l1) < 1e-4
        assert torch.allclose(e, e1, atol=1e-5) and torch.allclose(n, n1, atol=1e-5)
        assert torch.allclose(o, o1[:, r * kl:(r + 1) * kl], atol=1e-5)
        assert torch.allclose(h, h1[r * vl:(r + 1) * vl], atol=1e-5)
