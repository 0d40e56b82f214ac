"""hccl_b200 -- a Blackwell-native collective communication library with HCCL's API surface.

Layout:
  hccl_b200.comm       Communicator (ctypes face of the C API in include/hccl/*.h)
  hccl_b200.ops        fused matmul+collective ops (MC2), MoE dispatch/combine, GEMM
  hccl_b200.parallel   torch ProcessGroup backend, tensor/data-parallel layers
  hccl_b200.models     Llama-style decoder used by the end-to-end benchmarks
  hccl_b200.utils      build helpers, clocks sampler, simulation harness
"""
from .types import DataType, ReduceOp, Engine, Result  # noqa: F401
from .comm import Communicator, get_root_info  # noqa: F401

__version__ = "0.1.0"
