"""Argument-blob / resource-context API of the fused-operator interface, and the graph-mode entry points with their
resource queries, on the simulation backend.

Reference behaviour: src/common/hccl_mc2.cc:21-165 (setter validation, context creation is idempotent per
(operator, algorithm config)); src/ops/interface_graph_mode/calc_resource_graph_mode.cc:47-94 (offline / online resource
estimates and algorithm selection from an opaque parameter object); src/ops/all_reduce/all_reduce_op.cc:58-103 (graph-mode
entry addressed by group name and tag).
"""
import ctypes

import numpy as np

from hccl_b200._lib import lib
from hccl_b200.types import DataType, Result
from hccl_b200.utils.sim import run_ranks

vp, u8, u32, u64 = ctypes.c_void_p, ctypes.c_uint8, ctypes.c_uint32, ctypes.c_uint64


class OpResCtx(ctypes.Structure):
    _fields_ = [("magic", u32), ("opType", u32), ("rank", u32), ("nranks", u32), ("srcDataType", u32), ("dstDataType", u32),
                ("reduceType", u32), ("commEngine", u32), ("count", u64), ("heapBytes", u64), ("heap", vp * 32), ("mcHeap", vp),
                ("workspaceOff", u64), ("workspaceBytes", u64), ("flagOff", u64), ("timeoutNs", u64), ("algConfig", ctypes.c_char * 128)]


class OpRes(ctypes.Structure):
    _fields_ = [("scratchBytes", u64), ("streamNum", u32), ("taskNum", u32), ("ctaNum", u32), ("algName", ctypes.c_char * 128), ("engine", u32)]


def _declare():
    l = lib()
    l.HcclKfcAllocOpArgs.argtypes = [ctypes.POINTER(vp)]
    l.HcclKfcFreeOpArgs.argtypes = [vp]
    l.HcclKfcOpArgsSetSrcDataType.argtypes = [vp, u8]
    l.HcclKfcOpArgsSetDstDataType.argtypes = [vp, u8]
    l.HcclKfcOpArgsSetReduceType.argtypes = [vp, u32]
    l.HcclKfcOpArgsSetCount.argtypes = [vp, u64]
    l.HcclKfcOpArgsSetAlgConfig.argtypes = [vp, ctypes.c_char_p]
    l.HcclKfcOpArgsSetCommEngine.argtypes = [vp, u8]
    l.HcclCreateOpResCtx.argtypes = [vp, u8, vp, ctypes.POINTER(vp)]
    for n in ("Create",):
        getattr(l, "HcclOpParamGraphMode" + n).argtypes = [ctypes.POINTER(vp)]
    l.HcclOpParamGraphModeDestroy.argtypes = [vp]
    l.HcclOpParamGraphModeSetOpType.argtypes = [vp, ctypes.c_int]
    l.HcclOpParamGraphModeSetDataCount.argtypes = [vp, u64]
    l.HcclOpParamGraphModeSetDataType.argtypes = [vp, ctypes.c_int]
    l.HcclOpParamGraphModeSetReduceOp.argtypes = [vp, ctypes.c_int]
    l.HcclOpParamGraphModeSetRoot.argtypes = [vp, u32]
    l.HcclOpParamGraphModeSetGroup.argtypes = [vp, ctypes.c_char_p]
    l.HcclCalcOpResOfflineGraphMode.argtypes = [vp, u32, ctypes.POINTER(OpRes)]
    l.HcclCalcOpResOnlineGraphMode.argtypes = [vp, vp, ctypes.POINTER(OpRes)]
    l.HcclSelectAlgGraphMode.argtypes = [vp, vp, ctypes.c_char_p, u32]
    tail = [ctypes.c_char_p, vp, ctypes.c_char_p, ctypes.POINTER(vp), u32, vp, u64]
    l.HcclAllReduceGraphMode.argtypes = [vp, vp, u64, ctypes.c_int, ctypes.c_int] + tail
    l.HcclAllGatherGraphMode.argtypes = [vp, vp, u64, ctypes.c_int] + tail
    l.HcclBroadcastGraphMode.argtypes = [vp, u64, ctypes.c_int, u32] + tail
    return l


def test_op_args_setters_validate():
    l = _declare()
    a = vp()
    assert l.HcclKfcAllocOpArgs(ctypes.byref(a)) == 0 and a.value
    assert l.HcclKfcOpArgsSetSrcDataType(a, int(DataType.BFP16)) == 0
    assert l.HcclKfcOpArgsSetDstDataType(a, int(DataType.FP32)) == 0
    assert l.HcclKfcOpArgsSetSrcDataType(a, 200) != 0
    assert l.HcclKfcOpArgsSetReduceType(a, 0) == 0 and l.HcclKfcOpArgsSetReduceType(a, 9) != 0
    assert l.HcclKfcOpArgsSetCount(a, 1 << 20) == 0
    assert l.HcclKfcOpArgsSetAlgConfig(a, b"AllGather=level0:fullmesh") == 0
    assert l.HcclKfcOpArgsSetAlgConfig(a, b"x" * 200) != 0                 # longer than the 128-character limit
    assert l.HcclKfcOpArgsSetAlgConfig(a, None) == Result.E_PTR
    assert l.HcclKfcOpArgsSetCommEngine(a, 3) == 0 and l.HcclKfcOpArgsSetCommEngine(a, 1) != 0   # only device engines
    assert l.HcclKfcOpArgsSetCount(None, 1) == Result.E_PTR
    junk = ctypes.create_string_buffer(256)
    assert l.HcclKfcOpArgsSetCount(ctypes.cast(junk, vp), 1) == Result.E_PTR   # not a blob made by the allocator
    assert l.HcclKfcFreeOpArgs(a) == 0


def test_resource_context_describes_the_symmetric_heap():
    l = _declare()

    def body(comm, rank):
        a = vp()
        l.HcclKfcAllocOpArgs(ctypes.byref(a))
        l.HcclKfcOpArgsSetSrcDataType(a, int(DataType.FP32))
        l.HcclKfcOpArgsSetDstDataType(a, int(DataType.FP32))
        l.HcclKfcOpArgsSetCount(a, 1000)
        l.HcclKfcOpArgsSetAlgConfig(a, b"mine")
        h = vp(comm.handle)
        ctx1, ctx2 = vp(), vp()
        assert l.HcclCreateOpResCtx(h, 6, a, ctypes.byref(ctx1)) == 0
        assert l.HcclCreateOpResCtx(h, 6, a, ctypes.byref(ctx2)) == 0
        assert ctx1.value == ctx2.value                                    # one context per (operator, algorithm config)
        assert l.HcclCreateOpResCtx(h, 0, a, ctypes.byref(ctx2)) == Result.E_PARA
        assert l.HcclCreateOpResCtx(h, 6, None, ctypes.byref(ctx2)) == Result.E_PTR
        l.HcclKfcOpArgsSetCommEngine(a, 4)
        assert l.HcclCreateOpResCtx(h, 6, a, ctypes.byref(ctx2)) == Result.E_UNAVAIL   # no multicast mapping on the host backend
        c = OpResCtx.from_address(ctx1.value)
        assert c.magic == 0x4332434D and c.rank == rank and c.nranks == comm.size and c.count == 1000
        assert c.workspaceBytes >= 1000 * 4 * comm.size + (64 << 10) and c.flagOff + (64 << 10) == c.workspaceOff + c.workspaceBytes
        # use it the way a custom kernel would: write my rank into every peer's window, then read what the peers wrote
        for r in range(comm.size):
            ctypes.c_uint32.from_address(c.heap[r] + c.workspaceOff + 4 * rank).value = 1000 + rank
        comm.barrier()
        comm.synchronize()
        got = [ctypes.c_uint32.from_address(c.heap[rank] + c.workspaceOff + 4 * r).value for r in range(comm.size)]
        flags_zero = all(ctypes.c_uint32.from_address(c.heap[rank] + c.flagOff + 4 * i).value == 0 for i in range(64))
        l.HcclKfcFreeOpArgs(a)
        return got, flags_zero

    for got, flags_zero in run_ranks(3, body):
        assert got == [1000, 1001, 1002] and flags_zero


def test_graph_mode_resource_queries_and_entry_points():
    l = _declare()
    p = vp()
    assert l.HcclOpParamGraphModeCreate(ctypes.byref(p)) == 0
    res = OpRes()
    assert l.HcclCalcOpResOfflineGraphMode(p, 8, ctypes.byref(res)) == Result.E_PARA      # no operator type set yet
    assert l.HcclOpParamGraphModeSetOpType(p, 2) == 0 and l.HcclOpParamGraphModeSetOpType(p, 0) == Result.E_PARA
    assert l.HcclOpParamGraphModeSetDataCount(p, 1 << 20) == 0
    assert l.HcclOpParamGraphModeSetDataType(p, 11) == 0 and l.HcclOpParamGraphModeSetDataType(p, 99) != 0
    assert l.HcclOpParamGraphModeSetReduceOp(p, 0) == 0
    assert l.HcclCalcOpResOfflineGraphMode(p, 8, ctypes.byref(res)) == 0
    assert res.taskNum >= 1 and res.ctaNum >= 1 and res.algName and res.engine in (3, 4) and res.scratchBytes > 0
    assert l.HcclCalcOpResOfflineGraphMode(p, 1, ctypes.byref(res)) == Result.E_PARA

    def body(comm, rank):
        h = vp(comm.handle)
        q = vp()
        l.HcclOpParamGraphModeCreate(ctypes.byref(q))
        l.HcclOpParamGraphModeSetOpType(q, 2)
        l.HcclOpParamGraphModeSetDataCount(q, 4096)
        l.HcclOpParamGraphModeSetDataType(q, 4)
        l.HcclOpParamGraphModeSetReduceOp(q, 0)
        name = comm.name.encode()
        assert l.HcclOpParamGraphModeSetGroup(q, name) == 0
        r1, r2 = OpRes(), OpRes()
        assert l.HcclCalcOpResOnlineGraphMode(h, q, ctypes.byref(r1)) == 0
        assert l.HcclCalcOpResOnlineGraphMode(None, q, ctypes.byref(r2)) == 0             # resolved through the group name
        alg = ctypes.create_string_buffer(128)
        assert l.HcclSelectAlgGraphMode(h, q, alg, 128) == 0
        assert r1.algName == r2.algName == alg.value and r1.engine == 1
        x = np.full(4096, rank + 1.0, np.float32)
        out = np.empty_like(x)
        assert l.HcclAllReduceGraphMode(x.ctypes.data, out.ctypes.data, 4096, 4, 0, name, None, b"step0_ar", None, 0, None, 0) == 0
        g = np.empty(4096 * comm.size, np.float32)
        assert l.HcclAllGatherGraphMode(x.ctypes.data, g.ctypes.data, 4096, 4, name, None, b"step0_ag", None, 0, None, 0) == 0
        b = x.copy()
        assert l.HcclBroadcastGraphMode(b.ctypes.data, 4096, 4, 1, name, None, b"step0_bc", None, 0, None, 0) == 0
        comm.synchronize()
        assert l.HcclAllReduceGraphMode(x.ctypes.data, out.ctypes.data, 4096, 4, 0, b"no_such_group", None, b"t", None, 0, None, 0) != 0
        assert l.HcclAllReduceGraphMode(x.ctypes.data, out.ctypes.data, 4096, 4, 0, name, None, None, None, 0, None, 0) == Result.E_PTR
        l.HcclOpParamGraphModeDestroy(q)
        return out[0], g[::4096].tolist(), b[0]

    for out, g, b in run_ranks(3, body):
        assert out == 6.0 and g == [1.0, 2.0, 3.0] and b == 2.0
    assert l.HcclOpParamGraphModeDestroy(p) == 0


def test_graph_mode_variable_count_entry_points():
    """AllGatherV / ReduceScatterV / AlltoAllV / AlltoAllVC through the graph-mode entries (group name, tag, helper streams and
    scratch in the tail), against numpy; and the argument checks that differ from the fixed-count forms."""
    l = _declare()
    tail = [ctypes.c_char_p, vp, ctypes.c_char_p, ctypes.POINTER(vp), u32, vp, u64]
    l.HcclAllGatherVGraphMode.argtypes = [vp, vp, u64, vp, vp, ctypes.c_int] + tail
    l.HcclReduceScatterVGraphMode.argtypes = [vp, vp, vp, vp, u64, ctypes.c_int, ctypes.c_int] + tail
    l.HcclAlltoAllVGraphMode.argtypes = [vp, vp, vp, ctypes.c_int, vp, vp, vp, ctypes.c_int] + tail
    l.HcclAlltoAllVCGraphMode.argtypes = [vp, vp, ctypes.c_int, vp, ctypes.c_int] + tail
    n = 3
    counts = np.array([5, 0, 1201], np.uint64)                      # per-rank block sizes of the gather / scatter forms
    displs = np.array([0, 5, 5], np.uint64)
    total = int(counts.sum())
    M = np.array([[2, 0, 7], [300, 1, 0], [4, 5, 6]], np.uint64)    # M[i][j]: elements rank i sends to rank j
    rng = np.random.default_rng(23)
    ag_in = [rng.standard_normal(int(counts[r])).astype(np.float32) for r in range(n)]
    rs_in = [rng.integers(-8, 9, size=total).astype(np.float32) for _ in range(n)]
    a2a_in = [rng.standard_normal(int(M[r].sum())).astype(np.float32) for r in range(n)]
    FP32, SUM = 4, 0

    def body(comm, rank):
        name = comm.name.encode()
        t = lambda tag: (name, None, tag, None, 0, None, 0)
        g = np.zeros(total, np.float32)
        x = ag_in[rank] if counts[rank] else np.zeros(1, np.float32)
        assert l.HcclAllGatherVGraphMode(x.ctypes.data, g.ctypes.data, int(counts[rank]), counts.ctypes.data, displs.ctypes.data, FP32, *t(b"agv")) == 0
        s = np.zeros(max(1, int(counts[rank])), np.float32)
        assert l.HcclReduceScatterVGraphMode(rs_in[rank].ctypes.data, counts.ctypes.data, displs.ctypes.data, s.ctypes.data, int(counts[rank]), FP32, SUM, *t(b"rsv")) == 0
        sc, rc = M[rank].copy(), M[:, rank].copy()
        sd = np.concatenate([[0], np.cumsum(sc)[:-1]]).astype(np.uint64)
        rd = np.concatenate([[0], np.cumsum(rc)[:-1]]).astype(np.uint64)
        o1 = np.zeros(int(rc.sum()), np.float32)
        assert l.HcclAlltoAllVGraphMode(a2a_in[rank].ctypes.data, sc.ctypes.data, sd.ctypes.data, FP32, o1.ctypes.data, rc.ctypes.data, rd.ctypes.data, FP32, *t(b"a2av")) == 0
        o2 = np.zeros(int(rc.sum()), np.float32)
        assert l.HcclAlltoAllVCGraphMode(a2a_in[rank].ctypes.data, M.ctypes.data, FP32, o2.ctypes.data, FP32, *t(b"a2avc")) == 0
        comm.synchronize()
        # argument checks: own count must agree with the array; a product reduction is refused; element sizes must agree
        assert l.HcclAllGatherVGraphMode(x.ctypes.data, g.ctypes.data, int(counts[rank]) + 1, counts.ctypes.data, displs.ctypes.data, FP32, *t(b"bad")) == Result.E_PARA
        assert l.HcclReduceScatterVGraphMode(rs_in[rank].ctypes.data, counts.ctypes.data, displs.ctypes.data, s.ctypes.data, int(counts[rank]), FP32, 1, *t(b"bad")) == Result.E_NOT_SUPPORT
        assert l.HcclAlltoAllVCGraphMode(a2a_in[rank].ctypes.data, M.ctypes.data, FP32, o2.ctypes.data, 3, *t(b"bad")) == Result.E_PARA      # fp16 on the receive side
        assert l.HcclAlltoAllVGraphMode(a2a_in[rank].ctypes.data, None, sd.ctypes.data, FP32, o1.ctypes.data, rc.ctypes.data, rd.ctypes.data, FP32, *t(b"bad")) == Result.E_PTR
        assert l.HcclAllGatherVGraphMode(x.ctypes.data, g.ctypes.data, int(counts[rank]), counts.ctypes.data, displs.ctypes.data, FP32,
                                         b"no_such_group", None, b"t", None, 0, None, 0) != 0
        return g, s[:int(counts[rank])], o1, o2

    res = run_ranks(n, body)
    want_g = np.concatenate(ag_in)
    want_rs = np.sum(np.stack(rs_in).astype(np.float64), axis=0)
    for rank, (g, s, o1, o2) in enumerate(res):
        assert np.array_equal(g, want_g)
        lo = int(displs[rank])
        assert np.array_equal(s.astype(np.float64), want_rs[lo:lo + int(counts[rank])])
        want = np.concatenate([a2a_in[src][int(M[src, :rank].sum()):int(M[src, :rank + 1].sum())] for src in range(n)])
        assert np.array_equal(o1, want) and np.array_equal(o2, want)
