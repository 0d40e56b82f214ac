"""Fused matmul + collective kernels with all ranks emulated on one GPU (one cooperative launch, blockIdx.y = rank),
against fp32 PyTorch references of the unfused computation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _rel(out, ref):
    return (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)


@pytest.mark.parametrize("nranks,m_local,N,K", [(2, 128, 256, 256), (4, 256, 512, 512), (2, 384, 768, 1024), (4, 128, 264, 320), (8, 128, 512, 256)])
def test_allgather_matmul(nranks, m_local, N, K):
    from hccl_b200.utils import emu
    ctas = 148 // nranks
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=(4 * nranks * m_local * K + (1 << 20))) as w:
        for it in range(3):   # repeated calls alternate the workspace halves and reuse the cleared counters
            a = [_mk((m_local, K), 10 * it + r) for r in range(nranks)]
            b = [_mk((N, K), 100 + 10 * it + r, 0.05) for r in range(nranks)]
            out = [torch.zeros(nranks * m_local, N, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.fused(0, a, b, out, m_local, N, K, ctas, comm_ctas=2) == 0
            full = torch.cat(a).float()
            for r in range(nranks):
                assert _rel(out[r], full @ b[r].float().t()) < 2e-2


@pytest.mark.parametrize("nranks,M,N,K", [(2, 256, 256, 256), (4, 512, 512, 384), (2, 512, 776, 512), (8, 1024, 520, 256)])
def test_matmul_reduce_scatter(nranks, M, N, K):
    from hccl_b200.utils import emu
    ctas = 148 // nranks
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=(4 * M * N + (1 << 20))) as w:
        for it in range(3):
            a = [_mk((M, K), 20 * it + r) for r in range(nranks)]
            b = [_mk((N, K), 200 + 20 * it + r, 0.05) for r in range(nranks)]
            out = [torch.zeros(M // nranks, N, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.fused(1, a, b, out, M, N, K, ctas) == 0
            # reference: bf16-rounded partials summed in fp32 (what the kernel does, in rank order)
            partial = [(a[r].float() @ b[r].float().t()).to(torch.bfloat16).float() for r in range(nranks)]
            ref = sum(partial)
            rows = M // nranks
            for r in range(nranks):
                assert _rel(out[r], ref[r * rows:(r + 1) * rows]) < 1e-2


@pytest.mark.parametrize("nranks,M,N,K", [(2, 128, 256, 256), (4, 128, 1024, 512), (4, 64, 512, 256), (2, 200, 256, 128), (8, 128, 1024, 256)])
def test_matmul_all_reduce(nranks, M, N, K):
    from hccl_b200.utils import emu
    ctas = min(148 // nranks, ((M + 127) // 128) * (N // 64))
    with emu.EmuWorld(nranks, 1 << 20, arena_bytes=(8 * M * N + (1 << 20))) as w:
        for it in range(3):
            a = [_mk((M, K), 30 * it + r) for r in range(nranks)]
            b = [_mk((N, K), 300 + 30 * it + r, 0.05) for r in range(nranks)]
            out = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.fused(2, a, b, out, M, N, K, ctas) == 0
            partial = [(a[r].float() @ b[r].float().t()).to(torch.bfloat16).float() for r in range(nranks)]
            ref = sum(partial)
            for r in range(nranks):
                assert _rel(out[r], ref) < 1e-2
                assert torch.equal(out[r], out[0])   # every rank holds identical bits
