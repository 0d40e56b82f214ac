"""What the library does after a wait has run out: operator retry, the task-exception dump, and the heartbeat's stuck report.
Every failure is made on the host with simulated ranks: a rank records an operator but never runs it (the others' waits run
out and return an error status), so nothing faults, traps or hangs. Follows the reference's rules for re-execution
(docs/zh/user_guide/hccl_env/HCCL_OP_RETRY_ENABLE.md: all ranks at the same operator, input not overwritten)."""
import ctypes
import os
import time

import numpy as np
import pytest

from hccl_b200._lib import HcclError, lib
from hccl_b200.types import Result
from hccl_b200.utils.sim import run_ranks


@pytest.fixture
def fault_env(monkeypatch):
    def set_env(**kw):
        for k, v in kw.items():
            monkeypatch.setenv(k, v)
        lib().HcclResetEnvConfigForTest()
    yield set_env
    for k in ("HCCL_OP_RETRY_ENABLE", "HCCL_OP_RETRY_PARAMS", "HCCL_DEVICE_WAIT_TIMEOUT_MS", "HCCL_HEARTBEAT_PERIOD_MS", "HCCL_STUCK_CHECK_MS",
              "HCCL_EXCEPTION_DUMP_DIR", "HCCL_DFS_CONFIG"):
        monkeypatch.delenv(k, raising=False)
    lib().HcclResetEnvConfigForTest()


def _fault_counters(comm):
    a, b, c = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
    assert lib().HcclGetFaultCounters(ctypes.c_void_p(comm.handle), ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)) == 0
    return {"retries": a.value, "stuck": b.value, "dumps": c.value}


def _wait_suspended(comm, seconds=10.0):
    t0 = time.time()
    while comm.status() == 0 and time.time() - t0 < seconds:
        time.sleep(0.02)
    return comm.status()


def test_operator_retry_reruns_the_operator_all_ranks_stopped_at(fault_env):
    fault_env(HCCL_OP_RETRY_ENABLE="L0:1,L1:1,L2:0", HCCL_OP_RETRY_PARAMS="MaxCnt:2,HoldTime:50,IntervalTime:50",
              HCCL_DEVICE_WAIT_TIMEOUT_MS="400", HCCL_HEARTBEAT_PERIOD_MS="50")

    def body(comm, rank):
        warm = np.ones(8, np.float32)
        comm.all_reduce(warm)
        comm.synchronize()
        x = np.full(1000, rank + 1.0, np.float32)
        y = np.zeros_like(x)
        if rank == 1:
            lib().HcclInjectOpDrop(ctypes.c_void_p(comm.handle), 1)      # this rank records the next operator but never runs it
        comm.all_reduce(x, y)
        if rank == 1:
            comm.synchronize()                       # nothing ran here, so nothing fails here
            assert _wait_suspended(comm) == 1        # the peers' timeout arrives with the heartbeat, before the next launch
        else:
            with pytest.raises(HcclError) as e:      # the wait for rank 1 runs out and is reported, not hung on
                comm.synchronize()
            assert e.value.code == Result.E_TIMEOUT
        # the next call finds the communicator suspended, with retry configured: the ranks agree and run the operator again
        z = np.ones(4, np.float32)
        comm.all_reduce(z)
        comm.synchronize()
        return y[0], y[-1], z[0], _fault_counters(comm)["retries"], comm.status()

    for y0, y1, z0, retries, status in run_ranks(3, body, timeout_s=60):
        assert (y0, y1, z0) == (6.0, 6.0, 3.0)
        assert retries == 1 and status == 0


def test_operator_retry_refuses_an_operator_whose_input_was_overwritten(fault_env):
    fault_env(HCCL_OP_RETRY_ENABLE="L0:1", HCCL_OP_RETRY_PARAMS="MaxCnt:1,HoldTime:20,IntervalTime:20", HCCL_DEVICE_WAIT_TIMEOUT_MS="300",
              HCCL_HEARTBEAT_PERIOD_MS="50")

    def body(comm, rank):
        x = np.full(64, rank + 1.0, np.float32)
        if rank == 0:
            lib().HcclInjectOpDrop(ctypes.c_void_p(comm.handle), 1)
        comm.all_reduce(x)                           # in place: a second run would add to partial sums
        try:
            comm.synchronize()
        except HcclError:
            pass
        assert _wait_suspended(comm) == 1
        with pytest.raises(HcclError) as e:
            comm.barrier()
        return e.value.code

    assert run_ranks(2, body, timeout_s=60) == [Result.E_OPRETRY_FAIL, Result.E_OPRETRY_FAIL]


def test_task_exception_dump_names_the_flags_that_are_behind(fault_env, tmp_path):
    fault_env(HCCL_DEVICE_WAIT_TIMEOUT_MS="300", HCCL_EXCEPTION_DUMP_DIR=str(tmp_path), HCCL_HEARTBEAT_PERIOD_MS="50")

    def body(comm, rank):
        for _ in range(3):
            w = np.ones(16, np.float32)
            comm.all_reduce(w)
            comm.synchronize()
        x = np.ones(256, np.float32)
        y = np.zeros_like(x)
        if rank == 1:
            lib().HcclInjectOpDrop(ctypes.c_void_p(comm.handle), 1)
        comm.all_reduce(x, y)
        code = 0
        try:
            comm.synchronize()
        except HcclError as e:
            code = e.code
        _wait_suspended(comm)
        stuck, exc = ctypes.create_string_buffer(1024), ctypes.create_string_buffer(8192)
        assert lib().HcclGetFaultReports(ctypes.c_void_p(comm.handle), stuck, len(stuck), exc, len(exc)) == 0
        return code, exc.value.decode(), _fault_counters(comm)["dumps"], comm.name

    res = run_ranks(2, body, timeout_s=60)
    code0, report0, dumps0, name = res[0]
    assert code0 == Result.E_TIMEOUT and dumps0 == 1
    assert "peer=1" in report0 and "host notifies from rank 1" in report0 and "last 4 operators" in report0 and "AllReduce" in report0
    assert res[1][2] == 0                                     # the rank that dropped the operator saw no exception of its own
    path = tmp_path / f"hccl_exception_{name}_rank0.bin"
    assert path.exists()
    buf = ctypes.create_string_buffer(1 << 16)
    assert lib().HcclReadExceptionDump(str(path).encode(), buf, len(buf)) == 0
    text = buf.value.decode()
    assert f"comm={name} rank=0/2 code=1 peer=1" in text and "operators=4" in text
    path.write_bytes(path.read_bytes()[:40])                  # a truncated file is reported, not read past its end
    assert lib().HcclReadExceptionDump(str(path).encode(), buf, len(buf)) == Result.E_PARA


def test_watchdog_reports_a_stuck_communicator_and_the_slowest_rank(fault_env):
    fault_env(HCCL_DEVICE_WAIT_TIMEOUT_MS="1500", HCCL_HEARTBEAT_PERIOD_MS="50", HCCL_STUCK_CHECK_MS="300")

    def body(comm, rank):
        x = np.ones(32, np.float32)
        y = np.zeros_like(x)
        if rank == 2:
            lib().HcclInjectOpDrop(ctypes.c_void_p(comm.handle), 1)
        comm.all_reduce(x, y)                         # ranks 0 and 1 wait for rank 2 for 1.5 s: long enough to be called stuck
        try:
            comm.synchronize()
        except HcclError:
            pass
        stuck = ctypes.create_string_buffer(1024)
        assert lib().HcclGetFaultReports(ctypes.c_void_p(comm.handle), stuck, len(stuck), None, 0) == 0
        return stuck.value.decode(), _fault_counters(comm)["stuck"]

    res = run_ranks(3, body, timeout_s=60)
    for rank in (0, 1):
        text, n = res[rank]
        assert n >= 1 and text.startswith("STUCK:") and f"rank {rank} has 0 of" in text and "no progress" in text
    assert res[2][1] == 0                             # nothing is in flight on the rank that skipped the operator


def test_task_monitor_interval_sets_the_sampling_period_of_the_watchdog(fault_env):
    """HCCL_DFS_CONFIG task_monitor_interval:<ms> is how often the watchdog samples progress. A wait of 0.9 s ends before the default
    period of one second has sampled twice, so no stuck report can be made from it; with 50 ms sampling a 300 ms stall is reported."""
    def run(dfs):
        env = dict(HCCL_DEVICE_WAIT_TIMEOUT_MS="900", HCCL_STUCK_CHECK_MS="300")
        if dfs:
            env["HCCL_DFS_CONFIG"] = dfs
        fault_env(**env)

        def body(comm, rank):
            x = np.ones(32, np.float32)
            y = np.zeros_like(x)
            if rank == 1:
                lib().HcclInjectOpDrop(ctypes.c_void_p(comm.handle), 1)
            comm.all_reduce(x, y)
            try:
                comm.synchronize()
            except HcclError:
                pass
            return _fault_counters(comm)["stuck"]

        return run_ranks(2, body, timeout_s=60)

    assert run("task_monitor_interval:50")[0] >= 1
    import os
    os.environ.pop("HCCL_DFS_CONFIG", None)
    assert run("")[0] == 0
