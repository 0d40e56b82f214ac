"""Environment-variable parsing: accepted forms, defaults, and rejection of malformed values.

Mirrors the reference's configuration unit tests (test/ut/common/ut_alg_env_config.cpp: each variable with valid, boundary
and invalid strings, resetting the parsed state between cases).
"""
import ctypes

import pytest

from hccl_b200._lib import lib
from hccl_b200.types import Result

ALL_VARS = ["HCCL_OP_EXPANSION_MODE", "HCCL_ALGO", "HCCL_ALGO_NAME", "HCCL_DETERMINISTIC", "HCCL_EXEC_TIMEOUT", "HCCL_DFS_CONFIG",
            "HCCL_OP_RETRY_ENABLE", "HCCL_OP_RETRY_PARAMS", "HCCL_BUFFSIZE", "HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", "HCCL_NVLS_ENABLE",
            "HCCL_MAX_CTAS", "HCCL_DEVICE_WAIT_TIMEOUT_MS", "HCCL_CONNECT_TIMEOUT", "HCCL_IF_BASE_PORT", "HCCL_IF_IP", "HCCL_TUNING_FILE",
            "HCCL_ENTRY_LOG_ENABLE", "HCCL_SOCKET_IFNAME"]


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for v in ALL_VARS:
        monkeypatch.delenv(v, raising=False)
    yield
    for v in ALL_VARS:
        monkeypatch.delenv(v, raising=False)
    lib().HcclResetEnvConfigForTest()


def describe():
    l = lib()
    l.HcclDescribeEnvConfig.argtypes = [ctypes.c_char_p, ctypes.c_uint32]
    l.HcclDescribeEnvConfig.restype = ctypes.c_int
    buf = ctypes.create_string_buffer(4096)
    rc = l.HcclDescribeEnvConfig(buf, 4096)
    d = dict(kv.split("=", 1) for kv in buf.value.decode().split(";") if "=" in kv) if rc == 0 else {}
    return rc, d


def test_defaults():
    rc, d = describe()
    assert rc == 0
    assert d["expansion"] == "DEFAULT" and d["algoSet"] == "0" and d["deterministic"] == "0"
    assert d["execTimeout"] == "1836" and d["bufferBytes"] == str(200 << 20) and d["deviceWaitMs"] == "20000"
    assert d["nvls"] == "1" and d["maxCtas"] == "0" and d["inconsistent"] == "1" and d["heartbeat"] == "1"


@pytest.mark.parametrize("value,want", [("SM", "SM"), ("NVLS", "NVLS"), ("COPY_ENGINE", "COPY_ENGINE"), ("HOST", "HOST"),
                                        ("AIV", "SM"), ("CCU_MS", "NVLS"), ("CCU_SCHED", "NVLS"), ("AI_CPU", "COPY_ENGINE"), ("AICPU_TS", "COPY_ENGINE")])
def test_expansion_mode_names_and_aliases(monkeypatch, value, want):
    monkeypatch.setenv("HCCL_OP_EXPANSION_MODE", value)
    rc, d = describe()
    assert rc == 0 and d["expansion"] == want


def test_expansion_mode_per_op_and_errors(monkeypatch):
    monkeypatch.setenv("HCCL_OP_EXPANSION_MODE", "allreduce:NVLS;allgather:SM")
    rc, d = describe()
    assert rc == 0 and d["expansion.AllReduce"] == "NVLS" and d["expansion.AllGather"] == "SM" and d["expansion"] == "DEFAULT"
    for bad in ("GPU", "allreduce:XPU", "nosuchop:SM"):
        monkeypatch.setenv("HCCL_OP_EXPANSION_MODE", bad)
        assert describe()[0] == Result.E_PARA


def test_hccl_algo_global_per_op_and_errors(monkeypatch):
    monkeypatch.setenv("HCCL_ALGO", "level0:NA;level1:ring")
    rc, d = describe()
    assert rc == 0 and d["algoSet"] == "1" and d["algo"].lower().startswith("na,ring")
    monkeypatch.setenv("HCCL_ALGO", "allreduce=level0:NA;level1:NHR/allgather=level0:NA;level1:fullmesh/others=level0:NA;level1:ring")
    rc, d = describe()
    assert rc == 0 and d["algo.AllReduce"].lower().startswith("na,nhr") and d["algo.AllGather"].lower().startswith("na,fullmesh")
    assert d["algo"].lower().startswith("na,ring")
    for bad in ("level0:warp", "level9:ring", "allreduce=level0", "frobnicate=level0:NA;level1:ring"):
        monkeypatch.setenv("HCCL_ALGO", bad)
        assert describe()[0] == Result.E_PARA, bad


def test_algo_name_override(monkeypatch):
    monkeypatch.setenv("HCCL_ALGO_NAME", "allreduce=InsAllReduceRing;allgather=InsAllGatherNHR")
    rc, d = describe()
    assert rc == 0 and d["algoName.AllReduce"] == "InsAllReduceRing" and d["algoName.AllGather"] == "InsAllGatherNHR"
    monkeypatch.setenv("HCCL_ALGO_NAME", "InsAllReduceRing")
    assert describe()[0] == Result.E_PARA


def test_deterministic(monkeypatch):
    for v, want in (("false", "0"), ("true", "1"), ("TRUE", "1"), ("strict", "2")):
        monkeypatch.setenv("HCCL_DETERMINISTIC", v)
        rc, d = describe()
        assert rc == 0 and d["deterministic"] == want
    monkeypatch.setenv("HCCL_DETERMINISTIC", "maybe")
    assert describe()[0] == Result.E_PARA


def test_exec_timeout_and_buffer_size(monkeypatch):
    monkeypatch.setenv("HCCL_EXEC_TIMEOUT", "77")
    monkeypatch.setenv("HCCL_BUFFSIZE", "64")
    rc, d = describe()
    assert rc == 0 and d["execTimeout"] == "77" and d["bufferBytes"] == str(64 << 20)
    for bad in ("abc", "-1", "12s"):
        monkeypatch.setenv("HCCL_EXEC_TIMEOUT", bad)
        assert describe()[0] == Result.E_PARA, bad
    monkeypatch.delenv("HCCL_EXEC_TIMEOUT")
    for bad in ("0", "99999999", "big"):
        monkeypatch.setenv("HCCL_BUFFSIZE", bad)
        assert describe()[0] == Result.E_PARA, bad


def test_dfs_config(monkeypatch):
    monkeypatch.setenv("HCCL_DFS_CONFIG", "cluster_heartbeat:off, stuck_detection:off, connection_fault_detection_time:30, task_monitor_interval:500, inconsistent_check:every")
    rc, d = describe()
    assert rc == 0 and d["heartbeat"] == "0" and d["stuck"] == "0" and d["faultDetect"] == "30" and d["monitorMs"] == "500" and d["inconsistent"] == "2"
    for bad in ("cluster_heartbeat", "cluster_heartbeat:perhaps", "connection_fault_detection_time:5", "unknown_key:on", "inconsistent_check:sometimes"):
        monkeypatch.setenv("HCCL_DFS_CONFIG", bad)
        assert describe()[0] == Result.E_PARA, bad


def test_op_retry(monkeypatch):
    monkeypatch.setenv("HCCL_OP_RETRY_ENABLE", "L0:1, L1:0, L2:1")
    monkeypatch.setenv("HCCL_OP_RETRY_PARAMS", "MaxCnt:3, HoldTime:6000, IntervalTime:500")
    rc, d = describe()
    assert rc == 0 and d["retry"] == "101" and d["retryMax"] == "3" and d["retryHold"] == "6000" and d["retryInterval"] == "500"
    monkeypatch.setenv("HCCL_OP_RETRY_ENABLE", "L0:2")
    assert describe()[0] == Result.E_PARA
    monkeypatch.setenv("HCCL_OP_RETRY_ENABLE", "L0:1")
    monkeypatch.setenv("HCCL_OP_RETRY_PARAMS", "MaxCnt:lots")
    assert describe()[0] == Result.E_PARA


def test_split_ratio_and_device_knobs(monkeypatch):
    monkeypatch.setenv("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", "3:1")
    monkeypatch.setenv("HCCL_NVLS_ENABLE", "0")
    monkeypatch.setenv("HCCL_MAX_CTAS", "24")
    monkeypatch.setenv("HCCL_DEVICE_WAIT_TIMEOUT_MS", "1500")
    monkeypatch.setenv("HCCL_IF_BASE_PORT", "61000")
    monkeypatch.setenv("HCCL_TUNING_FILE", "/nonexistent/table.txt")
    rc, d = describe()
    assert rc == 0 and d["split"] == "3:1" and d["nvls"] == "0" and d["maxCtas"] == "24" and d["deviceWaitMs"] == "1500"
    assert d["basePort"] == "61000" and d["tuningFile"] == "/nonexistent/table.txt"
    monkeypatch.setenv("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", "3")
    assert describe()[0] == Result.E_PARA


def test_bad_environment_fails_communicator_creation(monkeypatch):
    from hccl_b200._lib import HcclError
    from hccl_b200.comm import Communicator, get_root_info

    monkeypatch.setenv("HCCL_DETERMINISTIC", "maybe")
    lib().HcclResetEnvConfigForTest()
    with pytest.raises(HcclError) as e:
        Communicator.from_root_info(1, get_root_info(), 0, backend="sim")
    assert e.value.code == Result.E_PARA


def test_socket_ifname_selects_the_bootstrap_address(monkeypatch):
    """The four forms of the reference (prefix list, '=' exact names, '^' everything but); HCCL_IF_IP wins over it; a value that matches
    no interface with an IPv4 address is refused. The loopback interface exists everywhere, so it is what the cases name."""
    for spec in ("lo", "=lo", "nosuchprefix,lo", "^=nosuchname"):
        monkeypatch.setenv("HCCL_SOCKET_IFNAME", spec)
        rc, d = describe()
        assert rc == 0, spec
        if "nosuchname" not in spec:
            assert d["ifIp"] == "127.0.0.1", (spec, d["ifIp"])
        else:
            assert d["ifIp"].count(".") == 3
    monkeypatch.setenv("HCCL_SOCKET_IFNAME", "=lo")
    monkeypatch.setenv("HCCL_IF_IP", "10.1.2.3")
    rc, d = describe()
    assert rc == 0 and d["ifIp"] == "10.1.2.3"
    monkeypatch.delenv("HCCL_IF_IP")
    for spec in ("=nosuchname", "nosuchprefix", "^", "="):
        monkeypatch.setenv("HCCL_SOCKET_IFNAME", spec)
        rc, _ = describe()
        assert rc == Result.E_PARA, spec
