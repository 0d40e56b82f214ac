"""Communicator lifecycle, observability and host-side fault handling on the simulation backend.

Follows the reference's communicator / DFX tests (test/ut/framework/communicator/ut_hccl_api_base.cpp: init variants,
sub-communicators, names, buffers; op_common's last-op registry; the heartbeat and inconsistency checks of the DFS
configuration). Every failure here is made on the host: a rank that passes different arguments, a bootstrap message
that is dropped, a process that exits between operators.
"""
import ctypes
import json
import os
import subprocess
import sys
import threading

import numpy as np
import pytest

from hccl_b200._lib import HcclError, lib
from hccl_b200.comm import Communicator
from hccl_b200.types import Result
from hccl_b200.utils.sim import run_ranks

HERE = os.path.dirname(os.path.abspath(__file__))


class OpRecord(ctypes.Structure):
    _fields_ = [("seq", ctypes.c_uint64), ("opType", ctypes.c_uint32), ("dataType", ctypes.c_uint32), ("reduceOp", ctypes.c_uint32),
                ("root", ctypes.c_uint32), ("engine", ctypes.c_uint32), ("pad", ctypes.c_uint32), ("count", ctypes.c_uint64),
                ("algName", ctypes.c_char * 64), ("beginNs", ctypes.c_uint64), ("endNs", ctypes.c_uint64)]


def counters(comm):
    c = (ctypes.c_uint64 * 9)()
    assert lib().HcclGetCommCounters(ctypes.c_void_p(comm.handle), c) == 0
    return dict(zip(["ops", "bytes", "timeouts", "planCacheHits", "planCacheMisses", "fallbacks", "consistencyChecks", "chunkLoops", "kernelsLaunched"], c))


def test_rank_table_init(tmp_path, monkeypatch):
    port = 61000 + os.getpid() % 2000
    monkeypatch.setenv("HCCL_IF_BASE_PORT", str(port))
    lib().HcclResetEnvConfigForTest()
    table = {"status": "completed", "version": "1.0", "server_count": "1",
             "server_list": [{"server_id": "127.0.0.1", "device": [{"device_id": str(r), "rank_id": str(r)} for r in range(3)]}]}
    path = tmp_path / "ranktable.json"
    path.write_text(json.dumps(table))
    out = [None] * 3

    def body(r):
        comm = Communicator.from_cluster_info(str(path), r)
        x = np.full(64, r + 1.0, np.float32)
        comm.all_reduce(x)
        comm.synchronize()
        out[r] = (comm.size, x.copy())
        comm.destroy()

    th = [threading.Thread(target=body, args=(r,)) for r in range(3)]
    [t.start() for t in th]
    [t.join(120) for t in th]
    for r in range(3):
        assert out[r] is not None and out[r][0] == 3 and np.all(out[r][1] == 6.0)
    lib().HcclResetEnvConfigForTest()


@pytest.mark.parametrize("pods", [1, 2])
def test_rank_table_places_the_ranks_on_servers_and_super_pods(tmp_path, monkeypatch, pods):
    """On the host simulation the table's server_list (and super_pod_list) is what places the ranks: two servers of two ranks per pod give
    a two-level (with two pods: three-level) topology, and the multi-level executors serve the operators."""
    port = 63000 + os.getpid() % 1500 + pods
    monkeypatch.setenv("HCCL_IF_BASE_PORT", str(port))
    lib().HcclResetEnvConfigForTest()
    servers = 2 * pods
    n = servers * 2
    table = {"status": "completed", "version": "1.2", "server_count": str(servers),
             "server_list": [{"server_id": f"node_{s}", "device": [{"device_id": str(d), "rank_id": str(s * 2 + d)} for d in range(2)]} for s in range(servers)]}
    if pods > 1:
        table["super_pod_list"] = [{"super_pod_id": str(p), "server_list": [{"server_id": f"node_{p * 2 + k}"} for k in range(2)]} for p in range(pods)]
    path = tmp_path / "ranktable.json"
    path.write_text(json.dumps(table))
    out = [None] * n

    def body(r):
        comm = Communicator.from_cluster_info(str(path), r)
        desc = ctypes.create_string_buffer(1024)
        lib().HcclGetTopoDescription(ctypes.c_void_p(comm.handle), desc, 1024)
        x = np.full(5000, r + 1.0, np.float32)
        comm.all_reduce(x)
        comm.synchronize()
        alg = comm.last_algorithm()
        b = np.full(100, 7.0 if r == 3 else 0.0, np.float32)
        comm.broadcast(b, 3)
        comm.synchronize()
        out[r] = (desc.value.decode(), alg, comm.last_algorithm(), x[0], b[0])
        comm.destroy()

    th = [threading.Thread(target=body, args=(r,)) for r in range(n)]
    [t.start() for t in th]
    [t.join(120) for t in th]
    lib().HcclResetEnvConfigForTest()
    for r in range(n):
        assert out[r] is not None
        desc, alg, alg2, x0, b0 = out[r]
        assert f"pods={pods} servers={servers} ranksPerServer=2 levels={pods + 1}" in desc and "regular=1" in desc, desc
        assert "Sequence" in alg and "Sequence" in alg2, (alg, alg2)
        assert x0 == n * (n + 1) / 2 and b0 == 7.0


@pytest.mark.parametrize("mutate,code", [
    (lambda t: t.update(status="initializing"), Result.E_PARA),
    (lambda t: t.update(server_count="2"), Result.E_PARA),
    (lambda t: t["server_list"][0]["device"].append({"device_id": "9", "rank_id": "0"}), Result.E_PARA),      # duplicate rank
    (lambda t: t["server_list"][0]["device"].pop(0), Result.E_PARA),                                          # rank 0 missing
    (lambda t: t.pop("server_list"), Result.E_PARA),
])
def test_rank_table_errors(tmp_path, mutate, code):
    table = {"status": "completed", "version": "1.0", "server_count": "1",
             "server_list": [{"server_id": "127.0.0.1", "device": [{"device_id": str(r), "rank_id": str(r)} for r in range(2)]}]}
    mutate(table)
    path = tmp_path / "bad.json"
    path.write_text(json.dumps(table))
    with pytest.raises(HcclError) as e:
        Communicator.from_cluster_info(str(path), 1)
    assert e.value.code == code
    with pytest.raises(HcclError):
        Communicator.from_cluster_info(str(tmp_path / "missing.json"), 0)
    (tmp_path / "garbage.json").write_text("{not json")
    with pytest.raises(HcclError):
        Communicator.from_cluster_info(str(tmp_path / "garbage.json"), 0)


def test_sub_communicators_names_and_buffers():
    def body(comm, rank):
        assert comm.name.startswith("hccl_world_")
        addr, size = ctypes.c_void_p(), ctypes.c_uint64()
        assert lib().HcclGetHcclBuffer(ctypes.c_void_p(comm.handle), ctypes.byref(addr), ctypes.byref(size)) == 0
        assert addr.value and size.value == 4 << 20
        # two disjoint halves, each all-reducing its own data; then a single-member group
        members = [r for r in range(comm.size) if r % 2 == rank % 2]
        sub = comm.create_sub_comm(members, sub_id=100 + rank % 2)
        x = np.full(32, rank + 1.0, np.float32)
        sub.all_reduce(x)
        sub.synchronize()
        got = (sub.rank, sub.size, sub.name, x[0])
        sub.destroy()
        none = comm.create_sub_comm([0] if rank == 0 else None, sub_id=7)
        if rank == 0:
            assert none is not None and none.size == 1
            y = np.arange(5, dtype=np.float32)
            none.all_reduce(y)
            none.synchronize()
            assert np.array_equal(y, np.arange(5, dtype=np.float32))
            none.destroy()
        else:
            assert none is None
        # the parent still works after its children are gone
        z = np.ones(8, np.float32)
        comm.all_reduce(z)
        comm.synchronize()
        assert z[0] == comm.size
        return got

    res = run_ranks(4, body, buffer_mb=4)
    for r, (sr, ss, name, v) in enumerate(res):
        assert ss == 2 and sr == r // 2
        assert v == (1 + 3 if r % 2 == 0 else 2 + 4)
    assert res[0][2] == res[2][2] and res[1][2] == res[3][2] and res[0][2] != res[1][2]


def test_symmetric_allocation_and_peer_pointers():
    def body(comm, rank):
        h = ctypes.c_void_p(comm.handle)
        p = ctypes.c_void_p()
        assert lib().HcclCommSymAlloc(h, 4096, ctypes.byref(p)) == 0
        mine = (ctypes.c_uint32 * 1024).from_address(p.value)
        for i in range(1024):
            mine[i] = rank * 10000 + i
        comm.barrier()
        comm.synchronize()
        peer = ctypes.c_void_p()
        nxt = (rank + 1) % comm.size
        assert lib().HcclSymWinGetPeerPointer(h, p, nxt, ctypes.byref(peer)) == 0
        theirs = (ctypes.c_uint32 * 1024).from_address(peer.value)
        got = theirs[5]
        mc = ctypes.c_void_p()
        rc_mc = lib().HcclSymGetMulticastPointer(h, p, ctypes.byref(mc))
        bad = ctypes.c_void_p()
        rc_bad = lib().HcclSymWinGetPeerPointer(h, ctypes.c_void_p(0x10), nxt, ctypes.byref(bad))
        comm.barrier()
        comm.synchronize()
        assert lib().HcclCommSymFree(h, p) == 0
        assert lib().HcclCommSymFree(h, p) != 0          # double free is reported
        huge = ctypes.c_void_p()
        rc_huge = lib().HcclCommSymAlloc(h, 1 << 40, ctypes.byref(huge))
        return got, rc_mc, rc_bad, rc_huge

    for r, (got, rc_mc, rc_bad, rc_huge) in enumerate(run_ranks(3, body)):
        assert got == ((r + 1) % 3) * 10000 + 5
        assert rc_mc != 0                                  # the host backend has no multicast mapping
        assert rc_bad != 0 and rc_huge == 24      # HCCL_E_OOM


def test_counters_last_ops_histogram_selection_and_trace(tmp_path):
    def body(comm, rank):
        h = ctypes.c_void_p(comm.handle)
        x = np.ones(1000, np.float32)
        outs = [np.empty_like(x) for _ in range(3)]
        for o in outs:
            comm.all_reduce(x, o)
        g = np.empty(4000, np.float32)
        comm.all_gather(x, g)
        comm.synchronize()
        c = counters(comm)
        recs = (OpRecord * 16)()
        n = ctypes.c_uint32()
        assert lib().HcclGetLastOps(h, recs, 16, ctypes.byref(n)) == 0
        ops = [(recs[i].opType, recs[i].count, recs[i].algName.decode(), recs[i].endNs >= recs[i].beginNs) for i in range(n.value)]
        hist = ctypes.create_string_buffer(2048)
        assert lib().HcclGetAlgoHistogram(h, hist, 2048) == 0
        alg = ctypes.create_string_buffer(128)
        eng = ctypes.c_uint32()
        assert lib().HcclQuerySelection(h, 2, 1000, 4, 0, alg, 128, ctypes.byref(eng)) == 0
        topo = ctypes.create_string_buffer(512)
        assert lib().HcclGetTopoDescription(h, topo, 512) == 0
        path = str(tmp_path / f"trace_{rank}.json")
        assert lib().HcclDumpTrace(h, path.encode()) == 0
        small = ctypes.create_string_buffer(4)
        assert lib().HcclGetTopoDescription(h, small, 4) != 0      # a too-small buffer is an error, not an overrun
        return c, ops, hist.value.decode(), alg.value.decode(), eng.value, topo.value.decode(), path

    for c, ops, hist, alg, eng, topo, path in run_ranks(4, body):
        assert c["ops"] == 4 and c["bytes"] >= 4 * 4000 and c["timeouts"] == 0
        assert c["planCacheMisses"] >= 2 and c["planCacheHits"] >= 2        # the second and third all-reduce reuse the schedule
        assert c["consistencyChecks"] == 2                                 # first call per (op, dtype, reduce op)
        assert [o[0] for o in ops] == [2, 2, 2, 6] and all(o[3] for o in ops) and ops[0][1] == 1000
        assert ops[0][2] == alg and alg in hist and eng == 1                # host engine on the simulation backend
        assert "ranksPerServer=4" in topo
        trace = json.load(open(path))
        events = trace["traceEvents"] if isinstance(trace, dict) else trace
        assert len([e for e in events if e.get("ph") == "X"]) == 4


def test_tuning_table_text_round_trip():
    l = lib()
    l.HcclTuningTableLoadText.argtypes = [ctypes.c_char_p]
    assert l.HcclTuningTableReset() == 0
    text = b"# op nranks engine maxBytes alg ctas\nallreduce 8 SM 65536 SmAllReduceMesh1DOneShot 8\nallreduce 8 NVLS inf NvlsAllReduceTwoShot 32\n"
    assert l.HcclTuningTableLoadText(text) == 0
    buf = ctypes.create_string_buffer(4096)
    assert l.HcclTuningTableDump(buf, 4096) == 0
    dump = buf.value.decode()
    assert "SmAllReduceMesh1DOneShot" in dump and "NvlsAllReduceTwoShot" in dump and "65536" in dump
    assert l.HcclTuningTableLoadText(b"allreduce eight SM 1 X 1\n") != 0
    assert l.HcclTuningTableLoadText(b"allreduce 8 WARP 1 X 1\n") != 0
    assert l.HcclTuningTableReset() == 0
    assert l.HcclTuningTableDump(buf, 4096) == 0 and b"NvlsAllReduceTwoShot 32" not in buf.value


def test_algorithm_listing_and_log_counters():
    l = lib()
    buf = ctypes.create_string_buffer(4096)
    assert l.HcclListAlgorithms(2, buf, 4096) == 0
    names = buf.value.decode().split(";")
    assert {"InsAllReduceMesh1DOneShot", "InsAllReduceRing", "InsAllReduceNHR"} <= set(names)
    l.HcclGetLogRecordCount.restype = ctypes.c_uint64
    before = l.HcclGetLogRecordCount(3)
    assert l.HcclAllReduce(None, None, 8, 4, 0, None, None) != 0
    x = np.zeros(4, np.float32)

    def body(comm, rank):
        with pytest.raises(HcclError):
            comm.broadcast(x, 99)

    run_ranks(2, body)
    assert l.HcclGetLogRecordCount(3) > before            # errors are logged with their EI code, and counted


def test_suspend_resume_blocks_and_restores_operators():
    def body(comm, rank):
        x = np.ones(16, np.float32)
        comm.all_reduce(x)
        comm.synchronize()
        comm.barrier()
        comm.synchronize()
        comm.suspend()
        assert comm.status() == 1
        with pytest.raises(HcclError) as e:
            comm.all_reduce(x)
        assert e.value.code == Result.E_SUSPENDING
        comm.resume()                                      # collective: every rank resumes
        assert comm.status() == 0
        y = np.ones(16, np.float32)
        comm.all_reduce(y)
        comm.synchronize()
        return y[0]

    assert run_ranks(3, body) == [3.0, 3.0, 3.0]


def _steps_of(log, rank, phase):
    return [e.split(":")[2] for e in log.split(",") if e.startswith(f"{rank}:{phase}:")]


def test_destroy_and_resume_drain_the_device_before_the_host_barrier():
    """No rank may unmap memory (destroy) or clear its flags (resume) while a peer's kernel can still touch them: every rank
    drains its own device first, THEN all meet at the host barrier, and only then mappings and flags change."""
    buf = ctypes.create_string_buffer(1 << 16)
    lib().HcclTakeLifecycleLog(buf, len(buf))              # drop what earlier tests left

    def body(comm, rank):
        x = np.ones(16, np.float32)
        comm.all_reduce(x)
        comm.synchronize()
        comm.suspend()
        comm.resume()

    run_ranks(3, body)
    assert lib().HcclTakeLifecycleLog(buf, len(buf)) == 0
    log = buf.value.decode()
    for r in range(3):
        assert _steps_of(log, r, "resume") == ["quiesce", "barrier", "clear", "barrier"]
        assert _steps_of(log, r, "destroy") == ["quiesce", "barrier", "unmap"]
    # across ranks: every quiesce of a phase precedes every state change of that phase
    events = [e for e in log.split(",") if e]
    for phase, change in (("resume", "clear"), ("destroy", "unmap")):
        last_quiesce = max(i for i, e in enumerate(events) if e.endswith(f"{phase}:quiesce"))
        first_change = min(i for i, e in enumerate(events) if e.endswith(f"{phase}:{change}"))
        assert last_quiesce < first_change


def test_inconsistent_arguments_are_detected(monkeypatch):
    monkeypatch.setenv("HCCL_DFS_CONFIG", "inconsistent_check:every")
    lib().HcclResetEnvConfigForTest()

    def body(comm, rank):
        x = np.ones(100 if rank != 1 else 96, np.float32)     # rank 1 passes a different count
        try:
            comm.all_reduce(x)
            comm.synchronize()
            first = 0
        except HcclError as e:
            first = e.code
        try:
            comm.broadcast(np.ones(8, np.float32), 0 if rank != 2 else 1)   # rank 2 names a different root
            comm.synchronize()
            second = 0
        except HcclError as e:
            second = e.code
        z = np.ones(8, np.float32)
        comm.all_reduce(z)                                  # a consistent call afterwards still runs
        comm.synchronize()
        return first, second, z[0]

    try:
        for first, second, z in run_ranks(3, body):
            assert first != 0 and second != 0 and z == 3.0
    finally:
        monkeypatch.delenv("HCCL_DFS_CONFIG")
        lib().HcclResetEnvConfigForTest()


def test_dropped_bootstrap_message_times_out_on_every_rank(monkeypatch):
    monkeypatch.setenv("HCCL_CONNECT_TIMEOUT", "2")
    monkeypatch.setenv("HCCL_DFS_CONFIG", "inconsistent_check:every")
    lib().HcclResetEnvConfigForTest()

    def body(comm, rank):
        if rank == 1:
            lib().HcclInjectBootstrapDrop(ctypes.c_void_p(comm.handle), 1)
        x = np.ones(10, np.float32)
        try:
            comm.all_reduce(x)
            comm.synchronize()
            return 0
        except HcclError as e:
            return e.code

    try:
        codes = run_ranks(2, body)
        assert all(c in (Result.E_TIMEOUT, 13) for c in codes), codes      # timeout, or the transfer error of the half-open exchange
        assert Result.E_TIMEOUT in codes
    finally:
        monkeypatch.delenv("HCCL_CONNECT_TIMEOUT")
        monkeypatch.delenv("HCCL_DFS_CONFIG")
        lib().HcclResetEnvConfigForTest()


def test_lost_rank_is_detected_by_heartbeat_between_operators():
    """Rank 1 exits (without a goodbye) after the first operator; rank 0 learns of it from the heartbeat, its communicator
    turns to SUSPENDING and the next operator is refused on the host -- nothing is launched against a dead peer."""
    env = dict(os.environ, HCCL_HEARTBEAT_PERIOD_MS="100", HCCL_HEARTBEAT_LOST_MS="800")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29541",
           os.path.join(HERE, "mp_worker_fault.py")]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300, env=env)
    assert "survivor saw status=1 code=22" in res.stdout, res.stdout[-4000:]
