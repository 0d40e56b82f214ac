"""Block-scaled fp8 (MXFP8) kernels: the quantiser against a plain PyTorch restatement of its rule, the tcgen05 block-scaled
GEMM against an fp32 PyTorch product of the DEQUANTISED operands, and the three fused operators on emulated ranks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _wild(shape, seed, base=1.0):
    """bf16 data whose 1 x 32 blocks differ in magnitude by up to 2^12, so a wrong scale byte cannot hide."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    rows, k = shape
    x = torch.randn(rows, k // 32, 32, generator=g, device="cuda") * base
    e = torch.randint(-6, 7, (rows, k // 32, 1), generator=g, device="cuda").float()
    return (x * torch.exp2(e)).view(rows, k).to(torch.bfloat16)


def _rel(out, ref):
    return (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-12)


@pytest.mark.parametrize("rows,k", [(128, 128), (200, 256), (1024, 1024), (77, 384)])
def test_quantiser_matches_the_reference_rule(rows, k):
    from hccl_b200.ops import mxfp8 as mx
    x = _wild((rows, k), rows + k)
    x[0, :32] = 0                                   # an all-zero block
    x[1, 32:64] = 448.0 * 2.0 ** 3                  # a block at the top of a binade
    q = mx.quantize(x)
    torch.cuda.synchronize()
    ref = mx.quantize_reference(x)
    assert torch.equal(q.scales, ref.scales)
    assert torch.equal(q.payload, ref.payload)
    # the format loses at most 2^-3 of the block maximum: 3 mantissa bits round to nearest (2^-4), and a block whose scaled
    # maximum lands in (448, 512) saturates at 448
    d = mx.dequantize(q)
    blk = x.float().view(rows, k // 32, 32)
    err = (d.view(rows, k // 32, 32) - blk).abs().amax(2)
    assert bool((err <= blk.abs().amax(2) * 2.0 ** -3 + 1e-30).all())


@pytest.mark.parametrize("m,n,k,tile", [(128, 128, 128, 128), (128, 256, 256, 256), (256, 512, 1024, 128), (384, 768, 512, 256),
                                        (200, 264, 384, 128), (200, 264, 384, 256), (1024, 1024, 2048, 0), (4096, 4096, 512, 0),
                                        # 192-wide tiles: odd tiles start at row 64 of a scale atom; partial last tiles; a single tile
                                        (128, 192, 128, 192), (256, 384, 512, 192), (384, 960, 640, 192), (200, 264, 384, 192), (2048, 8192, 512, 192),
                                        # CTA pairs (2256 / 2192 = 256- / 192-wide pair tiles): one pair, an odd number of row blocks (the second CTA of
                                        # the last pair idles), partial tiles in both directions, many tiles per pair
                                        (256, 256, 128, 2256), (128, 256, 256, 2256), (384, 768, 512, 2256), (200, 264, 384, 2256), (4096, 4096, 512, 2256),
                                        (256, 192, 128, 2192), (384, 960, 640, 2192), (200, 264, 384, 2192), (2048, 8192, 512, 2192)])
def test_block_scaled_gemm_matches_fp32_product_of_dequantised_operands(m, n, k, tile):
    from hccl_b200.ops import gemm as g, mxfp8 as mx
    a, w = mx.quantize(_wild((m, k), 1 + m)), mx.quantize(_wild((n, k), 2 + n, 0.05))
    ref = mx.dequantize(a) @ mx.dequantize(w).t()
    out32 = mx.gemm(a, w, out_dtype=torch.float32, tile_n=tile)
    out16 = mx.gemm(a, w, tile_n=tile)
    torch.cuda.synchronize()
    g.check_error()
    assert _rel(out32, ref) < 2e-3
    assert _rel(out16, ref) < 1e-2


def test_block_scaled_gemm_every_scale_byte_is_used():
    """Scales that differ for every (row, K block): one row of A and one of B get huge scales in single blocks; a kernel that
    picked a neighbouring block's or row's scale would be off by orders of magnitude."""
    from hccl_b200.ops import mxfp8 as mx
    m, n, k = 256, 256, 512
    a, w = torch.ones(m, k, device="cuda"), torch.ones(n, k, device="cuda")
    for kb in range(k // 32):
        a[(7 * kb) % m, kb * 32:(kb + 1) * 32] *= 2.0 ** (kb % 11)
        w[(13 * kb + 5) % n, kb * 32:(kb + 1) * 32] *= 2.0 ** -(kb % 9)
    qa, qw = mx.quantize(a.to(torch.bfloat16)), mx.quantize(w.to(torch.bfloat16))
    ref = mx.dequantize(qa) @ mx.dequantize(qw).t()
    for tile in (128, 192, 256, 2256, 2192):
        out = mx.gemm(qa, qw, out_dtype=torch.float32, tile_n=tile)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("tile", [256, 192])
@pytest.mark.parametrize("nranks,m_local,N,K", [(2, 128, 256, 256), (4, 256, 512, 512), (2, 384, 776, 1024)])
def test_allgather_matmul_mxfp8(nranks, m_local, N, K, tile, monkeypatch):
    from hccl_b200.ops import mxfp8 as mx
    from hccl_b200.utils import emu
    monkeypatch.setenv("HCCL_MX_TILE_N", str(tile))
    ctas = 148 // nranks
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=(4 * nranks * m_local * K + (1 << 20))) as w:
        for it in range(3):
            a = [mx.quantize(_wild((m_local, K), 10 * it + r)) for r in range(nranks)]
            b = [mx.quantize(_wild((N, K), 100 + 10 * it + r, 0.05)) for r in range(nranks)]
            out = [torch.zeros(nranks * m_local, N, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.fused_mx(0, a, b, out, m_local, N, K, ctas, comm_ctas=2) == 0
            full = torch.cat([mx.dequantize(t) for t in a])
            for r in range(nranks):
                assert _rel(out[r], full @ mx.dequantize(b[r]).t()) < 1e-2


@pytest.mark.parametrize("tile", [256, 192])
@pytest.mark.parametrize("nranks,M,N,K", [(2, 256, 256, 256), (4, 512, 512, 384), (2, 512, 776, 256)])
def test_matmul_reduce_scatter_mxfp8(nranks, M, N, K, tile, monkeypatch):
    from hccl_b200.ops import mxfp8 as mx
    from hccl_b200.utils import emu
    monkeypatch.setenv("HCCL_MX_TILE_N", str(tile))
    ctas = 148 // nranks
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=(4 * M * N + (1 << 20))) as w:
        for it in range(2):
            a = [mx.quantize(_wild((M, K), 20 * it + r)) for r in range(nranks)]
            b = [mx.quantize(_wild((N, K), 200 + 20 * it + r, 0.05)) for r in range(nranks)]
            out = [torch.zeros(M // nranks, N, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.fused_mx(1, a, b, out, M, N, K, ctas) == 0
            partial = [(mx.dequantize(a[r]) @ mx.dequantize(b[r]).t()).to(torch.bfloat16).float() for r in range(nranks)]
            ref = sum(partial)
            rows = M // nranks
            for r in range(nranks):
                assert _rel(out[r], ref[r * rows:(r + 1) * rows]) < 1.5e-2


@pytest.mark.parametrize("nranks,M,N,K", [(2, 128, 256, 256), (4, 128, 1024, 512), (2, 200, 512, 128)])
def test_matmul_all_reduce_mxfp8(nranks, M, N, K):
    from hccl_b200.ops import mxfp8 as mx
    from hccl_b200.utils import emu
    ctas = min(148 // nranks, ((M + 127) // 128) * (N // 128))
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=(8 * M * N + (1 << 20))) as w:
        for it in range(2):
            a = [mx.quantize(_wild((M, K), 30 * it + r)) for r in range(nranks)]
            b = [mx.quantize(_wild((N, K), 300 + 30 * it + r, 0.05)) for r in range(nranks)]
            out = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.fused_mx(2, a, b, out, M, N, K, ctas) == 0
            partial = [(mx.dequantize(a[r]) @ mx.dequantize(b[r]).t()).to(torch.bfloat16).float() for r in range(nranks)]
            ref = sum(partial)
            for r in range(nranks):
                assert _rel(out[r], ref) < 1.5e-2
                assert torch.equal(out[r], out[0])
