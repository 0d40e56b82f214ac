"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 256, 512), (256, 512, 1024), (384, 768, 200 * 8), (1000, 264, 520),
                                   (128, 8192, 1024), (2048, 3584, 2048), (64, 64, 64)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_matches_fp32_reference(shape, out_dtype):
    from hccl_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.05).to(torch.bfloat16)
    out = gemm.gemm_bf16(a, w, out_dtype=out_dtype)
    torch.cuda.synchronize()
    gemm.check_error()
    ref = a.float() @ w.float().t()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert err / scale < tol, f"max err {err} vs scale {scale}"


def test_gemm_back_to_back_is_deterministic():
    from hccl_b200.ops import gemm
    a = torch.randn(512, 1024, device="cuda").to(torch.bfloat16)
    w = torch.randn(1024, 1024, device="cuda").to(torch.bfloat16)
    o1 = gemm.gemm_bf16(a, w)
    o2 = gemm.gemm_bf16(a, w)
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("shape", [(256, 256, 64), (256, 512, 512), (512, 768, 1024), (384, 520, 328), (1000, 264, 520), (2048, 3584, 2048),
                                   (100, 256, 128)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_cta_pair_variant(shape, out_dtype):
    """256 x 256 tiles on CTA pairs (tcgen05 cta_group::2): odd row-block counts, ragged N and K tails included."""
    from hccl_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 5 + N * 11 + K)
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.05).to(torch.bfloat16)
    out = gemm.gemm_bf16(a, w, out_dtype=out_dtype, variant=2)
    torch.cuda.synchronize()
    gemm.check_error()
    ref = a.float() @ w.float().t()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert err / scale < tol, f"max err {err} vs scale {scale}"
