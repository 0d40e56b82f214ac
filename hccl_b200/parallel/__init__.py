"""Parallelism on top of the communicator.

  process_group     torch.distributed backend "hccl" (importing this package registers it)
  tensor_parallel   Column / Row parallel linears and the SwiGLU MLP on the fused matmul + collective kernels
  data_parallel     bucketed gradient all-reduce overlapped with the backward pass
"""
from .process_group import register_backend  # noqa: F401
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP  # noqa: F401
from .data_parallel import DataParallel  # noqa: F401
