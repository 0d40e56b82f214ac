"""Model code used by the end-to-end benchmarks: a Llama-3-architecture decoder on the tensor / sequence-parallel layers."""
from .llama import Llama, LlamaConfig  # noqa: F401
