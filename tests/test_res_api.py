"""Communicator resource API (hccl_res.h) on the simulation backend: state callbacks, configuration read-back, keyed
blobs, memory registration, rank graph queries on flat and multi-server topologies, exchanged blobs."""
import ctypes

import numpy as np
import pytest

from hccl_b200._lib import HcclError, HcclCommConfig, lib
from hccl_b200.types import Result
from hccl_b200.utils.sim import run_ranks

vp, u32, u64 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64


class LinkInfo(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("layer", u32), ("bandwidthGBs", ctypes.c_double), ("peerAccess", u32)]


CB = ctypes.CFUNCTYPE(None, vp, ctypes.c_int)


def _decl():
    l = lib()
    l.HcclCommRegCommStateCallback.argtypes = [vp, CB, vp]
    l.HcclConfigGetInfo.argtypes = [vp, ctypes.POINTER(HcclCommConfig)]
    l.HcclGroupStatusGet.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int)]
    l.HcclEngineCtxCreate.argtypes = [vp, ctypes.c_char_p, ctypes.c_int, u64, ctypes.POINTER(vp)]
    l.HcclEngineCtxGet.argtypes = [vp, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(u64)]
    l.HcclEngineCtxCopy.argtypes = [vp, ctypes.c_char_p, vp, u64]
    l.HcclEngineCtxDestroy.argtypes = [vp, ctypes.c_char_p]
    l.HcclCommMemReg.argtypes = [vp, vp, u64, ctypes.POINTER(u64)]
    l.HcclCommMemDereg.argtypes = [vp, vp]
    l.HcclMemAlloc.argtypes = [vp, u64, ctypes.POINTER(vp)]
    l.HcclMemFree.argtypes = [vp, vp]
    l.HcclSetAllocatorComm.argtypes = [vp]
    l.HcclAllocHook.argtypes = [ctypes.c_longlong, ctypes.c_int, vp]
    l.HcclAllocHook.restype = vp
    l.HcclFreeHook.argtypes = [vp, ctypes.c_longlong, ctypes.c_int, vp]
    l.HcclFreeHook.restype = None
    l.HcclRankGraphGetLayers.argtypes = [vp, ctypes.POINTER(u32)]
    l.HcclRankGraphGetRanksByLayer.argtypes = [vp, u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]
    l.HcclRankGraphGetInstSizeListByLayer.argtypes = [vp, u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]
    l.HcclRankGraphGetTopoTypeByLayer.argtypes = [vp, u32, ctypes.POINTER(ctypes.c_int)]
    l.HcclRankGraphGetLinks.argtypes = [vp, u32, u32, ctypes.POINTER(LinkInfo)]
    l.HcclCommAddExchangeInfo.argtypes = [vp, ctypes.c_char_p, vp, u32]
    l.HcclCommGetExchangeInfo.argtypes = [vp, u32, ctypes.c_char_p, vp, ctypes.POINTER(u32)]
    return l


def test_state_callback_config_and_group_status():
    l = _decl()

    def body(comm, rank):
        seen = []
        cb = CB(lambda user, st: seen.append(st))
        h = vp(comm.handle)
        assert l.HcclCommRegCommStateCallback(h, cb, None) == 0
        cfg = HcclCommConfig()
        assert l.HcclConfigGetInfo(h, ctypes.byref(cfg)) == 0
        st = ctypes.c_int(-1)
        assert l.HcclGroupStatusGet(comm.name.encode(), ctypes.byref(st)) == 0 and st.value == 0
        assert l.HcclGroupStatusGet(b"no_such_group", ctypes.byref(st)) == Result.E_NOT_FOUND
        comm.barrier()
        comm.synchronize()
        comm.suspend()
        assert l.HcclGroupStatusGet(comm.name.encode(), ctypes.byref(st)) == 0 and st.value == 1
        comm.resume()
        return seen, cfg.hcclBufferSize, cfg.hcclBackend, cfg.hcclCommName.decode(), comm.name, cb

    for seen, buf_mb, backend, cfg_name, name, _cb in run_ranks(2, body, buffer_mb=3):
        assert seen == [1, 0]                     # SUSPENDING, then READY again
        assert buf_mb == 3 and backend == 1 and cfg_name == name


def test_engine_ctx_blobs_and_memory_registration():
    l = _decl()

    def body(comm, rank):
        h = vp(comm.handle)
        p, q, n = vp(), vp(), u64()
        assert l.HcclEngineCtxGet(h, b"plan", 0, ctypes.byref(p), ctypes.byref(n)) == Result.E_NOT_FOUND
        assert l.HcclEngineCtxCreate(h, b"plan", 0, 64, ctypes.byref(p)) == 0
        assert l.HcclEngineCtxCreate(h, b"plan", 0, 64, ctypes.byref(q)) == Result.E_PARA            # exists already
        src = (ctypes.c_uint8 * 64)(*range(64))
        assert l.HcclEngineCtxCopy(h, b"plan", src, 64) == 0
        assert l.HcclEngineCtxGet(h, b"plan", 0, ctypes.byref(q), ctypes.byref(n)) == 0 and n.value == 64
        got = bytes((ctypes.c_uint8 * 64).from_address(q.value))
        assert l.HcclEngineCtxDestroy(h, b"plan") == 0
        assert l.HcclEngineCtxGet(h, b"plan", 0, ctypes.byref(q), ctypes.byref(n)) == Result.E_NOT_FOUND
        sym, off, off2 = vp(), u64(), u64()
        assert l.HcclCommSymAlloc(h, 8192, ctypes.byref(sym)) == 0
        assert l.HcclCommMemReg(h, sym, 8192, ctypes.byref(off)) == 0
        assert l.HcclCommMemReg(h, vp(sym.value + 4096), 4096, ctypes.byref(off2)) == 0 and off2.value == off.value + 4096
        stack = (ctypes.c_uint8 * 16)()
        assert l.HcclCommMemReg(h, stack, 16, ctypes.byref(off2)) == Result.E_NOT_SUPPORT
        assert l.HcclCommMemDereg(h, sym) == 0 and l.HcclCommMemDereg(h, stack) == Result.E_NOT_FOUND
        return got, off.value

    res = run_ranks(2, body)
    assert res[0][0] == bytes(range(64))
    assert res[0][1] == res[1][1]                 # the window offset is the same on every rank


def test_registered_window_lifetime():
    """Register, deregister, re-register, overlap, free with a live registration, destroy with live registrations."""
    l = _decl()

    def body(comm, rank):
        h = vp(comm.handle)
        a, b, off = vp(), vp(), u64()
        assert l.HcclCommSymAlloc(h, 1 << 16, ctypes.byref(a)) == 0
        assert l.HcclCommSymAlloc(h, 1 << 16, ctypes.byref(b)) == 0
        assert l.HcclCommMemReg(h, a, 1 << 16, ctypes.byref(off)) == 0
        first = off.value
        assert l.HcclCommMemReg(h, a, 1 << 16, ctypes.byref(off)) == 0 and off.value == first          # twice is fine
        assert l.HcclCommMemReg(h, vp(a.value + 4096), 8192, ctypes.byref(off)) == 0                     # inside a window: fine
        assert l.HcclCommMemReg(h, vp(a.value + (1 << 16) - 4096), 8192, ctypes.byref(off)) == Result.E_PARA   # straddles its end
        assert l.HcclCommMemDereg(h, a) == 0
        assert l.HcclCommMemDereg(h, a) == Result.E_NOT_FOUND                                              # already gone
        assert l.HcclCommMemReg(h, vp(a.value + (1 << 16) - 4096), 8192, ctypes.byref(off)) == 0         # now a window of its own
        assert l.HcclCommMemReg(h, a, 1 << 16, ctypes.byref(off)) == Result.E_PARA                        # would overlap it
        assert l.HcclCommMemDereg(h, vp(a.value + (1 << 16) - 4096)) == 0
        assert l.HcclCommMemReg(h, a, 1 << 16, ctypes.byref(off)) == 0 and off.value == first            # re-registered
        # freeing the allocation drops the windows inside it; the freed range can be allocated and registered again
        assert l.HcclCommSymFree(h, a) == 0
        assert l.HcclCommMemDereg(h, a) == Result.E_NOT_FOUND
        c2 = vp()
        assert l.HcclCommSymAlloc(h, 1 << 16, ctypes.byref(c2)) == 0 and c2.value == a.value
        assert l.HcclCommMemReg(h, c2, 1 << 16, ctypes.byref(off)) == 0 and off.value == first
        assert l.HcclCommMemReg(h, b, 1 << 16, ctypes.byref(off)) == 0
        second = off.value
        # operators still run with windows registered (on this backend they are staged as always) ...
        x = np.full(256, rank + 1.0, np.float32)
        comm.all_reduce(x)
        comm.synchronize()
        return first, second, float(x[0])      # ... and the communicator is destroyed with both windows still registered

    res = run_ranks(3, body)
    assert len({r[0] for r in res}) == 1 and len({r[1] for r in res}) == 1 and res[0][0] != res[0][1]
    assert all(r[2] == 6.0 for r in res)


def test_mem_alloc_is_a_registered_block_and_allocator_hooks_follow_the_attached_communicator():
    l = _decl()

    def body(comm, rank):
        h = vp(comm.handle)
        a, off = vp(), u64()
        assert l.HcclMemAlloc(h, 3000, ctypes.byref(a)) == 0
        assert l.HcclCommMemReg(h, a, 3000, ctypes.byref(off)) == 0            # already a window: registering again is fine
        first = off.value
        assert l.HcclMemFree(h, a) == 0
        assert l.HcclCommMemDereg(h, a) == Result.E_NOT_FOUND                   # the window went with the block
        assert l.HcclMemFree(h, a) == Result.E_NOT_FOUND
        if rank != 0:
            return first, None
        # allocator hooks: nothing attached -> NULL; attached -> registered blocks from that communicator's heap
        assert l.HcclSetAllocatorComm(None) == 0
        assert l.HcclAllocHook(4096, 0, None) is None
        assert l.HcclSetAllocatorComm(h) == 0
        p1, p2 = l.HcclAllocHook(4096, 0, None), l.HcclAllocHook(1 << 20, 0, None)
        assert p1 and p2 and p1 != p2
        assert l.HcclCommMemReg(h, vp(p2), 1 << 20, ctypes.byref(off)) == 0 and off.value > first
        l.HcclFreeHook(vp(p1), 4096, 0, None)
        assert l.HcclAllocHook(4096, 0, None) == p1                             # first fit: the freed block comes back
        assert l.HcclAllocHook(1 << 40, 0, None) is None                        # heap exhausted -> NULL, not an exception
        return first, p2

    res = run_ranks(2, body)
    assert res[0][0] == res[1][0]
    # the attached communicator is gone: the hooks do nothing and hand out nothing
    l.HcclFreeHook(vp(res[0][1]), 1 << 20, 0, None)
    assert l.HcclAllocHook(4096, 0, None) is None
    assert l.HcclSetAllocatorComm(vp(12345)) == Result.E_PTR


def test_python_wrappers_for_registered_memory():
    def body(comm, rank):
        p = comm.mem_alloc(1 << 16)
        q = comm.mem_alloc(4096)
        assert p and q and p != q
        comm.mem_free(q)
        assert comm.mem_alloc(4096) == q                      # first fit: the freed block comes back
        comm.mem_free(q)
        comm.mem_free(p)
        with pytest.raises(HcclError):
            comm.mem_free(p)                                  # already returned
        return p

    res = run_ranks(2, body)
    assert res[0] and res[1]


def test_cta_cap_is_a_per_communicator_setting():
    l = _decl()
    l.HcclCommSetMaxCtas.argtypes = [vp, u32]

    def body(comm, rank):
        comm.set_max_ctas(8)
        x = np.full(1000, rank + 1.0, np.float32)
        comm.all_reduce(x)                                    # operators keep working under a cap (the host engine ignores it)
        comm.synchronize()
        comm.set_max_ctas(0)
        return float(x[0])

    assert run_ranks(2, body) == [3.0, 3.0]
    assert l.HcclCommSetMaxCtas(vp(12345), 4) == Result.E_PTR


def test_rank_graph_flat_and_exchange_info():
    l = _decl()

    def body(comm, rank):
        h = vp(comm.handle)
        layers = u32()
        assert l.HcclRankGraphGetLayers(h, ctypes.byref(layers)) == 0
        ranks, n = (u32 * 8)(), u32(8)
        assert l.HcclRankGraphGetRanksByLayer(h, 0, ranks, ctypes.byref(n)) == 0
        small = u32(1)
        assert l.HcclRankGraphGetRanksByLayer(h, 0, ranks, ctypes.byref(small)) == Result.E_MEMORY and small.value == 3
        sizes, ns = (u32 * 4)(), u32(4)
        assert l.HcclRankGraphGetInstSizeListByLayer(h, 0, sizes, ctypes.byref(ns)) == 0
        t = ctypes.c_int(-1)
        assert l.HcclRankGraphGetTopoTypeByLayer(h, 0, ctypes.byref(t)) == 0
        assert l.HcclRankGraphGetTopoTypeByLayer(h, 5, ctypes.byref(t)) == Result.E_PARA
        link = LinkInfo()
        assert l.HcclRankGraphGetLinks(h, rank, (rank + 1) % 3, ctypes.byref(link)) == 0
        mine = f"hello from {rank}".encode()
        assert l.HcclCommAddExchangeInfo(h, b"greeting", mine, len(mine)) == 0
        buf, blen = ctypes.create_string_buffer(64), u32(64)
        assert l.HcclCommGetExchangeInfo(h, (rank + 1) % 3, b"greeting", buf, ctypes.byref(blen)) == 0
        return layers.value, list(ranks[: n.value]), list(sizes[: ns.value]), (link.type, link.layer, link.peerAccess), buf.raw[: blen.value].decode()

    for r, (layers, ranks, sizes, link, msg) in enumerate(run_ranks(3, body)):
        assert layers == 1 and ranks == [0, 1, 2] and sizes == [3]
        assert link == (3, 0, 1)                  # shared memory between simulated ranks, layer 0, directly addressable
        assert msg == f"hello from {(r + 1) % 3}"
