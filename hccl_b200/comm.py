"""Python face of the C API: `Communicator` wraps an `HcclComm` handle and accepts torch tensors or numpy arrays.

With CUDA tensors the ops are enqueued on `torch.cuda.current_stream()` (or the stream passed in); with host buffers the
communicator runs on the simulation backend and `synchronize()` drains its worker queue.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

from . import _lib
from ._lib import HcclCommConfig, HcclRootInfo, HcclSendRecvItem, check, lib
from .types import DataType, ReduceOp, from_numpy, from_torch


def get_root_info() -> bytes:
    info = HcclRootInfo()
    check(lib().HcclGetRootInfo(ctypes.byref(info)), "HcclGetRootInfo")
    return ctypes.string_at(ctypes.byref(info), _lib.HCCL_ROOT_INFO_BYTES)


def _root_from_bytes(b: bytes) -> HcclRootInfo:
    info = HcclRootInfo()
    ctypes.memmove(ctypes.byref(info), b, _lib.HCCL_ROOT_INFO_BYTES)
    return info


_TORCH_TENSOR = None


def _describe(buf):
    """-> (pointer, numel, DataType, is_cuda)"""
    global _TORCH_TENSOR
    if buf is None:
        return None, 0, DataType.INT8, False
    if _TORCH_TENSOR is None:
        import torch

        _TORCH_TENSOR = torch.Tensor
    if isinstance(buf, _TORCH_TENSOR):
        if not buf.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return buf.data_ptr(), buf.numel(), from_torch(buf.dtype), buf.is_cuda
    if hasattr(buf, "ctypes"):  # numpy
        if not buf.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return buf.ctypes.data, buf.size, from_numpy(buf.dtype), False
    raise TypeError(f"unsupported buffer type {type(buf)}")


_FN = {}


def _LIBFN(name):
    fn = _FN.get(name)
    if fn is None:
        fn = _FN[name] = getattr(lib(), name)
    return fn


_CUR_STREAM = None


def _current_stream_ptr() -> int:
    """Raw handle of torch's current CUDA stream without constructing a Stream object."""
    global _CUR_STREAM
    if _CUR_STREAM is None:
        import torch

        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        if raw is not None:
            _CUR_STREAM = lambda: raw(torch.cuda.current_device())
        else:
            _CUR_STREAM = lambda: torch.cuda.current_stream().cuda_stream
    return _CUR_STREAM()


def _u64_array(vals: Sequence[int]):
    return (ctypes.c_uint64 * len(vals))(*[int(v) for v in vals])


class Communicator:
    def __init__(self, handle: int):
        self._h = ctypes.c_void_p(handle)
        r, n = ctypes.c_uint32(), ctypes.c_uint32()
        check(lib().HcclGetRankId(self._h, ctypes.byref(r)), "HcclGetRankId")
        check(lib().HcclGetRankSize(self._h, ctypes.byref(n)), "HcclGetRankSize")
        self.rank, self.size = r.value, n.value

    # ---- construction -------------------------------------------------------------------------------------
    @classmethod
    def from_root_info(cls, nranks: int, root_info: bytes, rank: int, *, buffer_mb: int = 0, backend: str = "auto",
                       deterministic: Optional[int] = None, engine: int = 0, name: str = "",
                       exec_timeout_s: int = 0) -> "Communicator":
        cfg = HcclCommConfig()
        lib().HcclCommConfigInit(ctypes.byref(cfg))
        cfg.hcclBufferSize = buffer_mb
        cfg.hcclBackend = {"auto": 0, "sim": 1, "cuda": 2}[backend]
        if deterministic is not None:
            cfg.hcclDeterministic = int(deterministic)
        cfg.hcclOpExpansionMode = int(engine)
        cfg.hcclExecTimeoutSec = exec_timeout_s
        if name:
            cfg.hcclCommName = name.encode()
        info = _root_from_bytes(root_info)
        h = ctypes.c_void_p()
        check(lib().HcclCommInitRootInfoConfig(nranks, ctypes.byref(info), rank, ctypes.byref(cfg), ctypes.byref(h)),
              "HcclCommInitRootInfoConfig")
        return cls(h.value)

    @classmethod
    def from_cluster_info(cls, path: str, rank: int) -> "Communicator":
        h = ctypes.c_void_p()
        check(lib().HcclCommInitClusterInfo(path.encode(), rank, ctypes.byref(h)), "HcclCommInitClusterInfo")
        return cls(h.value)

    @classmethod
    def from_torch_process_group(cls, group=None, **kw) -> "Communicator":
        """Bootstraps over an existing torch.distributed group (any backend): rank 0's root info is broadcast as bytes."""
        import torch.distributed as dist

        rank, size = dist.get_rank(group), dist.get_world_size(group)
        obj = [get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls.from_root_info(size, obj[0], rank, **kw)

    def create_sub_comm(self, ranks: Optional[Sequence[int]], sub_id: int) -> Optional["Communicator"]:
        sub = ctypes.c_void_p()
        parent = ctypes.c_void_p(self._h.value)
        if ranks is None or self.rank not in ranks:
            check(lib().HcclCreateSubCommConfig(ctypes.byref(parent), 0, None, sub_id, 0, None, ctypes.byref(sub)), "HcclCreateSubCommConfig")
            return None
        arr = (ctypes.c_uint32 * len(ranks))(*ranks)
        check(lib().HcclCreateSubCommConfig(ctypes.byref(parent), len(ranks), arr, sub_id, list(ranks).index(self.rank), None,
                                            ctypes.byref(sub)), "HcclCreateSubCommConfig")
        return Communicator(sub.value)

    def destroy(self) -> None:
        if self._h is not None and self._h.value:
            check(lib().HcclCommDestroy(self._h), "HcclCommDestroy")
            self._h = None

    # ---- helpers --------------------------------------------------------------------------------------------
    @property
    def handle(self) -> int:
        return self._h.value

    @property
    def name(self) -> str:
        buf = ctypes.create_string_buffer(128)
        check(lib().HcclGetCommName(self._h, buf), "HcclGetCommName")
        return buf.value.decode()

    def _stream(self, is_cuda: bool, stream):
        if not is_cuda:
            return None
        if stream is None:
            return _current_stream_ptr()
        return getattr(stream, "cuda_stream", stream)

    def synchronize(self) -> None:
        check(lib().HcclSimStreamSynchronize(self._h), "HcclSimStreamSynchronize")

    def status(self) -> int:
        s = ctypes.c_int()
        check(lib().HcclCommGetStatus(self._h, ctypes.byref(s)), "HcclCommGetStatus")
        return s.value

    def async_error(self) -> int:
        e = ctypes.c_int()
        check(lib().HcclGetCommAsyncError(self._h, ctypes.byref(e)), "HcclGetCommAsyncError")
        return e.value

    def suspend(self) -> None:
        check(lib().HcclCommSuspend(self._h), "HcclCommSuspend")

    def resume(self) -> None:
        check(lib().HcclCommResume(self._h), "HcclCommResume")

    # ---- collectives ----------------------------------------------------------------------------------------
    def all_reduce(self, send, recv=None, op: ReduceOp = ReduceOp.SUM, stream=None) -> None:
        sp, n, dt, cu = _describe(send)
        rp = sp if recv is None or recv is send else _describe(recv)[0]
        rc = _LIBFN("HcclAllReduce")(sp, rp, n, dt, int(op), self._h, self._stream(cu, stream))
        if rc:
            check(rc, "HcclAllReduce")

    def broadcast(self, buf, root: int, stream=None) -> None:
        p, n, dt, cu = _describe(buf)
        check(lib().HcclBroadcast(p, n, dt, root, self._h, self._stream(cu, stream)), "HcclBroadcast")

    def reduce_scatter(self, send, recv, op: ReduceOp = ReduceOp.SUM, stream=None) -> None:
        sp, _, dt, cu = _describe(send)
        rp, n, _, _ = _describe(recv)
        check(lib().HcclReduceScatter(sp, rp, n, dt, int(op), self._h, self._stream(cu, stream)), "HcclReduceScatter")

    def reduce_scatter_v(self, send, send_counts, send_displs, recv, op: ReduceOp = ReduceOp.SUM, stream=None) -> None:
        sp, _, dt, cu = _describe(send)
        rp, n, _, cu2 = _describe(recv)
        sc, sd = _u64_array(send_counts), _u64_array(send_displs)
        check(lib().HcclReduceScatterV(sp, sc, sd, rp, int(send_counts[self.rank]), dt, int(op), self._h, self._stream(cu or cu2, stream)),
              "HcclReduceScatterV")

    def scatter(self, send, recv, root: int, stream=None) -> None:
        sp, _, _, _ = _describe(send)
        rp, n, dt, cu = _describe(recv)
        check(lib().HcclScatter(sp, rp, n, dt, root, self._h, self._stream(cu, stream)), "HcclScatter")

    def all_gather(self, send, recv, stream=None) -> None:
        sp, n, dt, cu = _describe(send)
        rp, _, _, _ = _describe(recv)
        check(lib().HcclAllGather(sp, rp, n, dt, self._h, self._stream(cu, stream)), "HcclAllGather")

    def all_gather_v(self, send, recv, recv_counts, recv_displs, stream=None) -> None:
        sp, n, dt, cu = _describe(send)
        rp, _, dt2, cu2 = _describe(recv)
        rc, rd = _u64_array(recv_counts), _u64_array(recv_displs)
        check(lib().HcclAllGatherV(sp, int(recv_counts[self.rank]), rp, rc, rd, dt2 if send is None else dt, self._h,
                                   self._stream(cu or cu2, stream)), "HcclAllGatherV")

    def reduce(self, send, recv, root: int, op: ReduceOp = ReduceOp.SUM, stream=None) -> None:
        sp, n, dt, cu = _describe(send)
        rp, _, _, _ = _describe(recv)
        check(lib().HcclReduce(sp, rp, n, dt, int(op), root, self._h, self._stream(cu, stream)), "HcclReduce")

    def all_to_all(self, send, recv, stream=None) -> None:
        sp, n, dt, cu = _describe(send)
        rp, m, dt2, _ = _describe(recv)
        check(lib().HcclAlltoAll(sp, n // self.size, dt, rp, m // self.size, dt2, self._h, self._stream(cu, stream)), "HcclAlltoAll")

    def all_to_all_v(self, send, send_counts, sdispls, recv, recv_counts, rdispls, stream=None) -> None:
        sp, _, dt, cu = _describe(send)
        rp, _, dt2, cu2 = _describe(recv)
        if send is None:
            dt = dt2
        if recv is None:
            dt2 = dt
        check(lib().HcclAlltoAllV(sp, _u64_array(send_counts), _u64_array(sdispls), dt, rp, _u64_array(recv_counts), _u64_array(rdispls),
                                  dt2, self._h, self._stream(cu or cu2, stream)), "HcclAlltoAllV")

    def all_to_all_vc(self, send, count_matrix, recv, stream=None) -> None:
        sp, _, dt, cu = _describe(send)
        rp, _, dt2, cu2 = _describe(recv)
        if send is None:
            dt = dt2
        if recv is None:
            dt2 = dt
        flat = [int(v) for row in count_matrix for v in row]
        check(lib().HcclAlltoAllVC(sp, _u64_array(flat), dt, rp, dt2, self._h, self._stream(cu or cu2, stream)), "HcclAlltoAllVC")

    def send(self, buf, dst: int, stream=None) -> None:
        p, n, dt, cu = _describe(buf)
        check(lib().HcclSend(p, n, dt, dst, self._h, self._stream(cu, stream)), "HcclSend")

    def recv(self, buf, src: int, stream=None) -> None:
        p, n, dt, cu = _describe(buf)
        check(lib().HcclRecv(p, n, dt, src, self._h, self._stream(cu, stream)), "HcclRecv")

    def batch_send_recv(self, items: Sequence[tuple], stream=None) -> None:
        """items: ("send"|"recv", buffer, peer)"""
        arr = (HcclSendRecvItem * len(items))()
        any_cuda = False
        for i, (kind, buf, peer) in enumerate(items):
            p, n, dt, cu = _describe(buf)
            any_cuda = any_cuda or cu
            arr[i].sendRecvType = 0 if kind == "send" else 1
            arr[i].buf = p
            arr[i].count = n
            arr[i].dataType = int(dt)
            arr[i].remoteRank = peer
        check(lib().HcclBatchSendRecv(arr, len(items), self._h, self._stream(any_cuda, stream)), "HcclBatchSendRecv")

    def barrier(self, stream=None, cuda: Optional[bool] = None) -> None:
        if cuda is None:
            cuda = self.is_cuda
        check(lib().HcclBarrier(self._h, self._stream(cuda, stream)), "HcclBarrier")

    # ---- symmetric memory and registered windows -----------------------------------------------------------------
    def sym_tensor(self, numel: int, dtype, register: bool = True):
        """A CUDA tensor over a fresh symmetric allocation (the same heap offset on every rank when all ranks make the same
        sequence of calls). With `register`, the range is also registered as a window, which lets AllReduce, ReduceScatter,
        AllGather and Broadcast on it run without staging through the scratch buffer."""
        import torch

        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        ptr = ctypes.c_void_p()
        check(lib().HcclCommSymAlloc(self._h, max(nbytes, 16), ctypes.byref(ptr)), "HcclCommSymAlloc")
        if register:
            off = ctypes.c_uint64()
            fn = lib().HcclCommMemReg
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64)]
            check(fn(self._h, ptr, max(nbytes, 16), ctypes.byref(off)), "HcclCommMemReg")

        class _Window:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr.value, False), "version": 3, "strides": None}

        t = torch.as_tensor(_Window(), device="cuda").view(dtype)
        t._hccl_sym_ptr = ptr.value
        return t

    def sym_free(self, tensor) -> None:
        """Returns a sym_tensor's memory to the arena (its window registration goes with it). Collective in the same sense as
        the allocation: every rank frees in the same order."""
        check(lib().HcclCommSymFree(self._h, ctypes.c_void_p(tensor._hccl_sym_ptr)), "HcclCommSymFree")

    def set_max_ctas(self, n: int) -> None:
        """Caps the grid of this communicator's collective kernels (0 = their own heuristics). A collective that overlaps compute,
        such as a gradient all-reduce during the backward pass, wants few CTAs so that the GEMMs keep their SMs."""
        check(lib().HcclCommSetMaxCtas(self._h, ctypes.c_uint32(n)), "HcclCommSetMaxCtas")

    def mem_alloc(self, nbytes: int) -> int:
        """Address of a fresh registered block of the symmetric heap (HcclMemAlloc); same calling rules as sym_tensor."""
        ptr = ctypes.c_void_p()
        fn = lib().HcclMemAlloc
        fn.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_void_p)]
        check(fn(self._h, nbytes, ctypes.byref(ptr)), "HcclMemAlloc")
        return ptr.value

    def mem_free(self, ptr: int) -> None:
        check(lib().HcclMemFree(self._h, ctypes.c_void_p(ptr)), "HcclMemFree")

    def mem_pool(self):
        """A torch.cuda.MemPool whose segments are registered blocks of this communicator's symmetric heap:

            pool = comm.mem_pool()
            with torch.cuda.use_mem_pool(pool):
                grads = torch.empty(n, dtype=torch.bfloat16, device="cuda")     # every rank, same order
            comm.all_reduce(grads, grads)            # runs on the window directly, no staging copy

        One communicator per process can serve the hooks at a time. Every rank has to make the same allocations in the same
        order inside the pool (segments are cut from the heap by a deterministic first-fit), as with NCCL's registered pools.
        Keep the pool alive as long as tensors from it are."""
        import torch
        from ._lib import LIB_PATH

        check(lib().HcclSetAllocatorComm(self._h), "HcclSetAllocatorComm")
        alloc = torch.cuda.memory.CUDAPluggableAllocator(str(LIB_PATH), "HcclAllocHook", "HcclFreeHook")
        return torch.cuda.MemPool(alloc.allocator())

    def last_algorithm(self) -> str:
        """Name of the algorithm the most recent operator ran with."""
        class Rec(ctypes.Structure):
            _fields_ = [("seq", ctypes.c_uint64), ("opType", ctypes.c_uint32), ("dataType", ctypes.c_uint32), ("reduceOp", ctypes.c_uint32),
                        ("root", ctypes.c_uint32), ("engine", ctypes.c_uint32), ("pad", ctypes.c_uint32), ("count", ctypes.c_uint64),
                        ("algName", ctypes.c_char * 64), ("beginNs", ctypes.c_uint64), ("endNs", ctypes.c_uint64)]
        recs = (Rec * 64)()
        n = ctypes.c_uint32()
        fn = lib().HcclGetLastOps
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint32)]
        check(fn(self._h, recs, 64, ctypes.byref(n)), "HcclGetLastOps")
        return recs[n.value - 1].algName.decode() if n.value else ""

    @property
    def is_cuda(self) -> bool:
        fn = getattr(lib(), "HcclCommIsCuda", None)
        if fn is None:
            return False
        fn.argtypes = [ctypes.c_void_p]
        fn.restype = ctypes.c_int
        return bool(fn(self._h))


_LIVE_STORES = []


def _store_exchange_root_info(rank: int, world: int) -> bytes:
    """Shares rank 0's root info through a torch TCPStore on MASTER_ADDR:(MASTER_PORT + 17)."""
    import os
    from datetime import timedelta

    from torch.distributed import TCPStore

    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + 17
    store = TCPStore(host, port, world, is_master=(rank == 0), timeout=timedelta(seconds=120), wait_for_workers=False)
    _LIVE_STORES.append(store)   # the server side lives in rank 0: keep it until the process exits
    key = "hccl_b200_root_info_" + os.environ.get("HCCL_B200_COMM_EPOCH", "0")
    if rank == 0:
        store.set(key, get_root_info())
    return store.get(key)


def init_from_env(**kw) -> Communicator:
    """One process per GPU, launched by torchrun (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT).

    Selects cuda:LOCAL_RANK when CUDA is available, shares the root info through torch.distributed if it is already
    initialised (any backend) or through a TCPStore otherwise, and returns the communicator."""
    import os

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if torch.cuda.is_available() and kw.get("backend", "auto") != "sim":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank % max(1, torch.cuda.device_count()))))
        torch.cuda.init()
        torch.zeros(1, device="cuda")   # create the context before the native library asks for the current device
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return Communicator.from_torch_process_group(None, **kw)
    root = _store_exchange_root_info(rank, world) if world > 1 else get_root_info()
    return Communicator.from_root_info(world, root, rank, **kw)
