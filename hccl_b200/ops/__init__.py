"""Fused compute + collective operators and their single-GPU building blocks."""
from .gemm import gemm_bf16  # noqa: F401
