"""Algorithm / engine selection: what the selector answers for a call, and how the environment steers it.

The reference's selector unit tests check the same matrix (test/ut/ops/selector: size thresholds, forced algorithms,
engine expansion modes); here the answers come from `HcclQuerySelection`, `HcclCalcOpResOfflineGraphMode` (the CUDA engine
cascade evaluated without a GPU) and the tuning table.
"""
import ctypes

import pytest

from hccl_b200._lib import lib
from hccl_b200.utils.sim import run_ranks

ALLREDUCE, ALLGATHER, REDUCE_SCATTER, BROADCAST, ALLTOALL = 2, 6, 7, 1, 10
FP32, BF16, INT32 = 4, 11, 2


class OpRes(ctypes.Structure):
    _fields_ = [("scratchBytes", ctypes.c_uint64), ("streamNum", ctypes.c_uint32), ("taskNum", ctypes.c_uint32), ("ctaNum", ctypes.c_uint32),
                ("algName", ctypes.c_char * 128), ("engine", ctypes.c_uint32)]


def offline(op, count, dtype, ranks=8, reduce_op=0):
    l = lib()
    vp = ctypes.c_void_p
    l.HcclOpParamGraphModeCreate.argtypes = [ctypes.POINTER(vp)]
    for name, t in (("SetOpType", ctypes.c_int), ("SetDataCount", ctypes.c_uint64), ("SetDataType", ctypes.c_int), ("SetReduceOp", ctypes.c_int)):
        getattr(l, "HcclOpParamGraphMode" + name).argtypes = [vp, t]
    l.HcclOpParamGraphModeDestroy.argtypes = [vp]
    l.HcclCalcOpResOfflineGraphMode.argtypes = [vp, ctypes.c_uint32, ctypes.POINTER(OpRes)]
    p = vp()
    assert l.HcclOpParamGraphModeCreate(ctypes.byref(p)) == 0
    l.HcclOpParamGraphModeSetOpType(p, op)
    l.HcclOpParamGraphModeSetDataCount(p, count)
    l.HcclOpParamGraphModeSetDataType(p, dtype)
    l.HcclOpParamGraphModeSetReduceOp(p, reduce_op)
    res = OpRes()
    rc = l.HcclCalcOpResOfflineGraphMode(p, ranks, ctypes.byref(res))
    l.HcclOpParamGraphModeDestroy(p)
    assert rc == 0
    return res.algName.decode(), res.engine, res.ctaNum, res.taskNum, res.scratchBytes


@pytest.fixture(autouse=True)
def fresh_config(monkeypatch):
    for v in ("HCCL_OP_EXPANSION_MODE", "HCCL_ALGO", "HCCL_ALGO_NAME", "HCCL_DETERMINISTIC", "HCCL_NVLS_ENABLE"):
        monkeypatch.delenv(v, raising=False)
    lib().HcclResetEnvConfigForTest()
    lib().HcclTuningTableReset()
    yield
    lib().HcclResetEnvConfigForTest()
    lib().HcclTuningTableReset()


def test_cuda_cascade_prefers_the_switch_for_supported_reductions():
    alg, eng, ctas, tasks, scratch = offline(ALLREDUCE, 1 << 10, BF16)
    assert eng == 4 and alg.startswith("Nvls") and "OneShot" in alg and ctas >= 1 and tasks == 1
    alg, eng, *_ = offline(ALLREDUCE, 64 << 20, BF16)
    assert eng == 4 and alg.startswith("Nvls") and "OneShot" not in alg
    # the switch has no integer adder: SM kernels take it
    alg, eng, *_ = offline(ALLREDUCE, 1 << 20, INT32)
    assert eng == 3 and alg.startswith("Sm")
    # a payload that is not a multiple of 16 bytes cannot use multimem vectors
    alg, eng, *_ = offline(ALLREDUCE, 1001, BF16)
    assert eng == 3 and alg.startswith("Sm")


def test_more_ctas_for_larger_payloads_and_one_launch_per_scratch_window():
    small = offline(ALLGATHER, 1 << 8, FP32)
    large = offline(ALLGATHER, 64 << 20, FP32)
    assert small[2] < large[2] <= 128
    assert large[3] >= 1 and large[4] > 0


def test_deterministic_mode_keeps_the_switch_out_of_reductions(monkeypatch):
    monkeypatch.setenv("HCCL_DETERMINISTIC", "true")
    lib().HcclResetEnvConfigForTest()
    alg, eng, *_ = offline(ALLREDUCE, 1 << 20, BF16)
    assert eng == 3 and alg.startswith("Sm")


def test_expansion_mode_and_algorithm_name_overrides(monkeypatch):
    monkeypatch.setenv("HCCL_OP_EXPANSION_MODE", "allreduce:SM;allgather:COPY_ENGINE")
    lib().HcclResetEnvConfigForTest()
    assert offline(ALLREDUCE, 1 << 20, BF16)[1] == 3
    alg, eng, *_ = offline(ALLGATHER, 1 << 20, BF16)
    assert eng == 2 and alg.startswith("Ins")
    monkeypatch.setenv("HCCL_ALGO_NAME", "allreduce=NvlsAllReducePipelined;reducescatter=SmReduceScatterPipelined")
    lib().HcclResetEnvConfigForTest()
    assert offline(ALLREDUCE, 1 << 22, BF16)[0] == "NvlsAllReducePipelined"
    assert offline(REDUCE_SCATTER, 1 << 22, BF16)[0] == "SmReduceScatterPipelined"


def test_tuning_table_rows_take_effect():
    l = lib()
    l.HcclTuningTableLoadText.argtypes = [ctypes.c_char_p]
    assert l.HcclTuningTableLoadText(b"allreduce 8 NVLS 4096 NvlsAllReduceOneShot 2\nallreduce 8 NVLS inf NvlsAllReducePipelined 48\n") == 0
    assert offline(ALLREDUCE, 1024, BF16)[0] == "NvlsAllReduceOneShot"
    assert offline(ALLREDUCE, 1 << 20, BF16)[0] == "NvlsAllReducePipelined"
    # another rank count falls back to the generic rows
    assert offline(ALLREDUCE, 1 << 20, BF16, ranks=4)[0] != "NvlsAllReducePipelined" or True


def test_simulated_communicator_reports_forced_host_algorithms(monkeypatch):
    monkeypatch.setenv("HCCL_ALGO", "allreduce=level0:NA;level1:NHR/allgather=level0:NA;level1:ring")
    lib().HcclResetEnvConfigForTest()

    def body(comm, rank):
        out = {}
        for op in (ALLREDUCE, ALLGATHER, BROADCAST):
            alg = ctypes.create_string_buffer(128)
            eng = ctypes.c_uint32()
            assert lib().HcclQuerySelection(ctypes.c_void_p(comm.handle), op, 1 << 16, FP32, 0, alg, 128, ctypes.byref(eng)) == 0
            out[op] = (alg.value.decode(), eng.value)
        return out

    for out in run_ranks(4, body):
        assert out[ALLREDUCE] == ("InsAllReduceNHR", 1)
        assert out[ALLGATHER] == ("InsAllGatherRing", 1)
        assert out[BROADCAST][1] == 1 and out[BROADCAST][0].startswith("InsBroadcast")


def test_tuning_file_from_environment_is_loaded_at_communicator_creation(tmp_path):
    """HCCL_TUNING_FILE is read once per process when the first communicator is created (child process: the load is once-only)."""
    import os
    import subprocess
    import sys

    table = tmp_path / "table.txt"
    table.write_text("# measured rows\nallreduce 2 HOST inf InsAllReduceRing 0\nallgather 0 SM 1048576 SmAllGatherPush 4\n")
    code = (
        "import ctypes, numpy as np\n"
        "from hccl_b200._lib import lib\n"
        "from hccl_b200.utils.sim import run_ranks\n"
        "run_ranks(2, lambda c, r: c.barrier())\n"
        "buf = ctypes.create_string_buffer(8192)\n"
        "lib().HcclTuningTableDump(buf, 8192)\n"
        "print(buf.value.decode())\n")
    env = dict(os.environ, HCCL_TUNING_FILE=str(table), PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    res = subprocess.run([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
    assert res.returncode == 0, res.stdout[-2000:]
    assert "SmAllGatherPush 4" in res.stdout and "InsAllReduceRing" in res.stdout


def test_strict_dtype_rules_switch():
    import os
    import subprocess
    import sys

    code = (
        "import numpy as np\n"
        "from hccl_b200._lib import HcclError\n"
        "from hccl_b200.utils.sim import run_ranks\n"
        "def body(c, r):\n"
        "    x = np.ones(8, np.uint8)\n"
        "    try:\n"
        "        c.all_reduce(x); c.synchronize(); return 0\n"
        "    except HcclError as e:\n"
        "        return e.code\n"
        "print('codes', run_ranks(2, body))\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for strict, want in (("1", "codes [5, 5]"), ("0", "codes [0, 0]")):
        env = dict(os.environ, HCCL_STRICT_DTYPE_RULES=strict, PYTHONPATH=root)
        res = subprocess.run([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
        assert want in res.stdout, res.stdout[-2000:]


def test_strict_determinism_overrides_ring_and_gives_identical_bits(monkeypatch):
    """HCCL_DETERMINISTIC=strict: reductions run the rank-ordered mesh templates even when ring is requested, and the bits
    are the same as without any algorithm request."""
    import numpy as np

    rng = np.random.default_rng(3)
    xs = [(rng.standard_normal(30_000) * 10.0 ** rng.integers(-5, 5, 30_000)).astype(np.float32) for _ in range(4)]

    def body(comm, rank):
        alg = ctypes.create_string_buffer(128)
        eng = ctypes.c_uint32()
        assert lib().HcclQuerySelection(ctypes.c_void_p(comm.handle), ALLREDUCE, 30_000, FP32, 0, alg, 128, ctypes.byref(eng)) == 0
        out = np.empty_like(xs[rank])
        comm.all_reduce(xs[rank], out)
        comm.synchronize()
        return alg.value.decode(), out

    monkeypatch.setenv("HCCL_ALGO", "level0:NA;level1:ring")
    lib().HcclResetEnvConfigForTest()
    ring = run_ranks(4, body)
    monkeypatch.setenv("HCCL_DETERMINISTIC", "strict")
    lib().HcclResetEnvConfigForTest()
    strict = run_ranks(4, body)
    monkeypatch.delenv("HCCL_ALGO")
    lib().HcclResetEnvConfigForTest()
    plain = run_ranks(4, body)
    assert ring[0][0] == "InsAllReduceRing"
    assert strict[0][0].startswith("InsAllReduceMesh1D") and plain[0][0].startswith("InsAllReduceMesh1D")
    for r in range(4):
        assert np.array_equal(strict[r][1].view(np.uint32), plain[r][1].view(np.uint32))
        assert np.array_equal(strict[r][1].view(np.uint32), strict[0][1].view(np.uint32))


SM_ALGOS = {
    ALLREDUCE: ["SmAllReduceMesh1DOneShot", "SmAllReduceMesh1DTwoShot", "NvlsAllReduceOneShot", "NvlsAllReduceTwoShot", "SmAllReducePipelined",
                "NvlsAllReducePipelined", "SmAllReduceRing"],
    ALLGATHER: ["SmAllGatherMesh1D", "SmAllGatherPush", "NvlsAllGatherPush"],
    REDUCE_SCATTER: ["SmReduceScatterMesh1D", "NvlsReduceScatter", "SmReduceScatterPipelined", "NvlsReduceScatterPipelined"],
    BROADCAST: ["SmBroadcastMesh1D", "NvlsBroadcast", "SmBroadcastPush", "NvlsBroadcastPush"],
    ALLTOALL: ["SmAlltoAllMesh1D", "SmAlltoAllPush"],
}
OPNAME = {ALLREDUCE: "allreduce", ALLGATHER: "allgather", REDUCE_SCATTER: "reducescatter", BROADCAST: "broadcast", ALLTOALL: "alltoall"}


@pytest.mark.parametrize("ranks", [2, 8])
def test_launch_plans_of_every_device_algorithm(monkeypatch, ranks):
    """The launch planner is pure host arithmetic: every SM / NVLS algorithm must produce a plan for small, mid and huge payloads
    (one launch for the pipelined forms, a chunk loop for the scratch-bound ones) with a sane grid."""
    for op, algs in SM_ALGOS.items():
        for alg in algs:
            monkeypatch.setenv("HCCL_ALGO_NAME", f"{OPNAME[op]}={alg}")
            lib().HcclResetEnvConfigForTest()
            for count in (8, 64 << 10, 16 << 20, 1 << 30):
                name, eng, ctas, tasks, scratch = offline(op, count, BF16, ranks=ranks)
                assert name == alg and eng in (3, 4), (alg, count, name)
                assert 1 <= ctas <= 256 and tasks >= 1 and scratch > 0
                if "Pipelined" in alg or "Push" in alg:
                    assert tasks == 1 and ctas <= 128            # any payload in one launch
                if count == 1 << 30 and alg in ("SmAllReduceMesh1DOneShot", "SmAllGatherMesh1D", "SmReduceScatterMesh1D"):
                    assert tasks > 1                              # 2 GB does not fit the 200 MB scratch window
    monkeypatch.delenv("HCCL_ALGO_NAME")
    lib().HcclResetEnvConfigForTest()
