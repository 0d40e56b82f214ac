"""Registers this library as the torch.distributed backend "hccl".

    import hccl_b200.parallel            # registers the backend
    dist.init_process_group("hccl", ...) # or "cpu:gloo,cuda:hccl"

CUDA tensors run on the CUDA communicator (SM / NVLS kernels over NVLink), CPU tensors on the host simulation backend, so
the same script works on a GPU-less machine. The binding is the in-tree C++ extension `hccl_b200/lib/hccl_b200_torch.so`
(built by `hccl_b200.utils.build.build_torch_ext()`); there is no Python fallback.
"""
from __future__ import annotations

import importlib.util
from pathlib import Path

import torch.distributed as dist

from .. import _lib

_EXT = None
EXT_PATH = Path(__file__).resolve().parents[1] / "lib" / "hccl_b200_torch.so"


def _ext():
    global _EXT
    if _EXT is None:
        _lib.lib()   # libhccl_b200.so first (RTLD_GLOBAL), the extension links against it
        if not EXT_PATH.exists():
            raise RuntimeError(f"{EXT_PATH} is missing: build it with `python -m hccl_b200.utils.build`")
        spec = importlib.util.spec_from_file_location("hccl_b200_torch", str(EXT_PATH))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _EXT = mod
    return _EXT


def _create(store, rank, size, timeout):
    return _ext().create_process_group(store, rank, size, timeout)


_registered = False


def register_backend() -> None:
    global _registered
    if _registered:
        return
    dist.Backend.register_backend("hccl", _create, devices=["cpu", "cuda"])
    _registered = True


register_backend()


def mem_pool():
    """A torch.cuda.MemPool whose segments are registered blocks of the symmetric heap of this process's "hccl" CUDA communicator
    (the one created by the group's first CUDA collective; run one before calling this). Tensors created under it need no staging
    copy in AllReduce / ReduceScatter / AllGather / Broadcast from 1 MB up:

        dist.all_reduce(torch.zeros(1, device="cuda"))                  # creates the communicator
        pool = hccl_b200.parallel.process_group.mem_pool()
        with torch.cuda.use_mem_pool(pool):
            ddp = DistributedDataParallel(model, device_ids=[dev])       # its gradient buckets become registered windows

    Every rank has to make the same allocations in the same order inside the pool. Set HCCL_SYM_HEAP_MB above what the pool will hold."""
    import ctypes

    import torch

    l = _lib.lib()
    h = ctypes.c_void_p()
    l.HcclGetAllocatorComm.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    if l.HcclGetAllocatorComm(ctypes.byref(h)) != 0 or not h.value:
        raise RuntimeError("no CUDA communicator yet: run one collective on a CUDA tensor through the hccl group first")
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(_lib.LIB_PATH), "HcclAllocHook", "HcclFreeHook")
    return torch.cuda.MemPool(alloc.allocator())
