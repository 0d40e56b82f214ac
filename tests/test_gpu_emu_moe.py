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


def _moe_quant_reference(x):
    """The dispatch kernel's block rule in plain PyTorch: per 1 x 32 block the smallest power-of-two scale with amax / scale <= 448,
    values divided by it and rounded to e4m3; returns the dequantised fp32 tensor, the e4m3 bytes and the e8m0 scale bytes."""
    T, H = x.shape
    v = x.float().view(T, H // 32, 32)
    amax = v.abs().amax(2)
    m, e = torch.frexp(amax / 448.0)                       # amax / 448 = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e)
    biased = torch.where(amax > 0, (e + 127).clamp(0, 254), torch.full_like(e, 127 - 8))
    scale = torch.exp2((biased - 127).float())
    q = (v / scale.unsqueeze(2)).to(torch.float8_e4m3fn)
    return (q.float() * scale.unsqueeze(2)).view(T, H), q.view(torch.uint8).view(T, H), biased.to(torch.uint8)


@pytest.mark.parametrize("nranks,T,E,K,H", [(2, 64, 8, 2, 256), (4, 200, 32, 4, 512), (4, 96, 64, 8, 1024)])
def test_mxfp8_dispatch_round_trip_matches_the_reference_quantiser(nranks, T, E, K, H):
    """Dispatch with the block-scaled payload (e4m3 + e8m0 scale per 32 values): the stand-in experts dequantise what they
    received, so every token must come back as (sum of its top-k weights) * dequantise(quantise(token)) -- the payload and the
    scales both have to be right, for blocks whose magnitudes differ by orders of magnitude."""
    from hccl_b200.ops import moe
    from hccl_b200.utils import emu
    l = moe._decl()
    cfg = moe.HcclMoeConfig(E, K, H, T, nranks * T * K, 1)
    g = torch.Generator(device="cuda").manual_seed(23)
    xs = []
    for _ in range(nranks):
        x = torch.randn(T, H // 32, 32, generator=g, device="cuda") * torch.exp2(torch.randint(-8, 9, (T, H // 32, 1), generator=g, device="cuda").float())
        x = x.view(T, H).to(torch.bfloat16)
        x[0, :32] = 0                                     # an all-zero block
        x[1, 32:64] = 448.0                               # a block exactly at the top of a binade
        xs.append(x.contiguous())
    idxs = [torch.topk(torch.randn(T, E, generator=g, device="cuda"), K, dim=1).indices.to(torch.int32).contiguous() for _ in range(nranks)]
    ws = [torch.rand(T, K, generator=g, device="cuda").contiguous() for _ in range(nranks)]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
    counts = [torch.zeros(E // nranks, dtype=torch.int32, device="cuda") for _ in range(nranks)]
    arena = (4 * nranks * T * K * H * 2 + (8 << 20))
    ctas = max(1, min(16, 148 // nranks))
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=arena) as w:
        arr = lambda ts: (ctypes.c_void_p * nranks)(*[t.data_ptr() for t in ts])
        for it in range(2):
            rc = l.HcclEmuMoeRoundTrip(w._h, ctypes.byref(cfg), arr(xs), arr(idxs), arr(ws), arr(outs), T, arr(counts), ctas)
            torch.cuda.synchronize()
            assert rc == 0
            for r in range(nranks):
                deq, _, _ = _moe_quant_reference(xs[r])
                # experts return bf16(dequantised); combine sums K weighted copies in fp32 and rounds to bf16 once more
                ref = deq.to(torch.bfloat16).float() * ws[r].sum(1, keepdim=True)
                err = (outs[r].float() - ref).abs() / (ref.abs() + 1e-30)
                assert float(err[ref.abs() > 0].max()) < 2.0 ** -6, float(err[ref.abs() > 0].max())
                assert bool((outs[r].float()[ref == 0] == 0).all())
                # and the format itself stays within e4m3's half-ulp (2^-4) of the block maximum
                blk = xs[r].float().view(T, H // 32, 32)
                assert bool(((deq.view(T, H // 32, 32) - blk).abs().amax(2) <= blk.abs().amax(2) * 2.0 ** -4 + 1e-30).all())
