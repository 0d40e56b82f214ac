"""Parallelism on top of the communicator: torch.distributed backend "hccl", tensor-parallel layers, data-parallel helpers."""
from .process_group import register_backend  # noqa: F401
