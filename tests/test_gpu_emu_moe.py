"""MoE dispatch + combine with all ranks emulated on one GPU (identity experts): every token must come back as
(sum of its top-k weights) * token, and the per-expert receive counts must equal the routing histogram."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nranks,T,E,K,H", [(2, 64, 8, 2, 256), (4, 300, 32, 4, 512), (4, 128, 64, 8, 1024), (8, 96, 64, 8, 256)])
def test_dispatch_combine_round_trip(nranks, T, E, K, H):
    from hccl_b200.ops import moe
    from hccl_b200.utils import emu
    l = moe._decl()
    cfg = moe.HcclMoeConfig(E, K, H, T, nranks * T * K, 0)
    g = torch.Generator(device="cuda").manual_seed(11)
    xs = [torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(nranks)]
    # skewed routing: a bias makes low expert ids more popular
    bias = -0.3 * torch.arange(E, device="cuda").float().log1p()
    idxs = [torch.topk(torch.randn(T, E, generator=g, device="cuda") + bias, K, dim=1).indices.to(torch.int32).contiguous() for _ in range(nranks)]
    ws = [torch.rand(T, K, generator=g, device="cuda").contiguous() for _ in range(nranks)]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
    counts = [torch.zeros(E // nranks, dtype=torch.int32, device="cuda") for _ in range(nranks)]
    arena = (4 * nranks * T * K * H * 2 + (8 << 20))
    ctas = max(1, min(16, 148 // nranks))
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=arena) as w:
        arr = lambda ts: (ctypes.c_void_p * nranks)(*[t.data_ptr() for t in ts])
        for it in range(2):   # the second round reuses buffers, flags and epochs
            rc = l.HcclEmuMoeRoundTrip(w._h, ctypes.byref(cfg), arr(xs), arr(idxs), arr(ws), arr(outs), T, arr(counts), ctas)
            torch.cuda.synchronize()
            assert rc == 0
            hist = torch.zeros(E, dtype=torch.int64, device="cuda")
            for r in range(nranks):
                hist += torch.bincount(idxs[r].flatten().long(), minlength=E)
            got = torch.cat(counts).long()
            assert torch.equal(got, hist)
            for r in range(nranks):
                ref = xs[r].float() * ws[r].sum(1, keepdim=True)
                err = (outs[r].float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
                assert err < 2e-2, err


def test_capacity_overflow_is_reported_not_written():
    from hccl_b200.ops import moe
    from hccl_b200.utils import emu
    l = moe._decl()
    nranks, T, E, K, H = 2, 64, 4, 2, 256
    cfg = moe.HcclMoeConfig(E, K, H, T, 16, 0)      # far too small a receive buffer
    xs = [torch.randn(T, H, device="cuda").to(torch.bfloat16) for _ in range(nranks)]
    idxs = [torch.zeros(T, K, dtype=torch.int32, device="cuda") + torch.tensor([0, 1], dtype=torch.int32, device="cuda") for _ in range(nranks)]
    ws = [torch.ones(T, K, device="cuda") for _ in range(nranks)]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=8 << 20) as w:
        arr = lambda ts: (ctypes.c_void_p * nranks)(*[t.data_ptr() for t in ts])
        rc = l.HcclEmuMoeRoundTrip(w._h, ctypes.byref(cfg), arr(xs), arr(idxs), arr(ws), arr(outs), T, None, 8)
        torch.cuda.synchronize()
        assert rc == 3     # HCCL_E_MEMORY: reported through the status word, no out-of-bounds write
