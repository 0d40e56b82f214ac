"""Host-side utilities that can be exercised without a GPU: the clock sampler against a fake NVML, the tuning-table generator."""
import json
import subprocess
import sys
import time
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_clock_sampler_reads_only_and_summarises(monkeypatch):
    calls = []
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlClocksEventReasonSwPowerCap = 0x4
    fake.nvmlClocksEventReasonHwSlowdown = 0x8
    fake.nvmlClocksEventReasonSwThermalSlowdown = 0x20
    fake.nvmlClocksEventReasonHwThermalSlowdown = 0x40
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, c: 1965
    clocks = iter([1965, 1500, 1300, 1310, 1290] + [1300] * 1000)
    fake.nvmlDeviceGetClockInfo = lambda h, c: next(clocks)
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4
    # anything that would SET a clock or a limit must never be called
    for name in ("nvmlDeviceSetGpuLockedClocks", "nvmlDeviceResetGpuLockedClocks", "nvmlDeviceSetPowerManagementLimit", "nvmlDeviceSetPersistenceMode",
                 "nvmlDeviceSetApplicationsClocks", "nvmlDeviceResetApplicationsClocks"):
        setattr(fake, name, lambda *a, _n=name: calls.append("FORBIDDEN " + _n))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    from hccl_b200.utils.clocks import ClockSampler

    s = ClockSampler(0, period_ms=1)
    s.start()
    time.sleep(0.02)
    s.mark()                       # warm-up samples are dropped
    time.sleep(0.05)
    out = s.stop()
    assert out["samples"] >= 5 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"]
    assert 1250 <= out["sm_mhz"] <= 1350
    assert not [c for c in calls if c.startswith("FORBIDDEN")]


def test_tuning_table_generator(tmp_path):
    rows = []
    for size, nvls_us, sm_us in [(1024, 10, 12), (4096, 11, 9), (65536, 20, 15), (1 << 20, 30, 40), (1 << 24, 100, 200)]:
        rows.append(dict(op="allreduce", dtype="bf16", ranks=8, bytes=size, ours_us=nvls_us, alg="NvlsAllReduceOneShot" if size < (1 << 20) else "NvlsAllReducePipelined"))
        rows.append(dict(op="allreduce", dtype="bf16", ranks=8, bytes=size, ours_us=sm_us, alg="SmAllReduceMesh1DOneShot"))
    f = tmp_path / "sweep.json"
    f.write_text(json.dumps(rows))
    res = subprocess.run([sys.executable, str(ROOT / "benchmarks" / "make_tuning_table.py"), "--ranks", "8", str(f)], stdout=subprocess.PIPE, text=True, check=True)
    lines = [l for l in res.stdout.splitlines() if l and not l.startswith("#")]
    assert lines == ["allreduce 8 NVLS 2048 NvlsAllReduceOneShot 0", "allreduce 8 NVLS 262144 none 0", "allreduce 8 NVLS inf NvlsAllReducePipelined 0",
                     "allreduce 8 SM inf SmAllReduceMesh1DOneShot 0"]
    # and the library accepts what the generator writes
    import ctypes

    from hccl_b200._lib import lib

    l = lib()
    l.HcclTuningTableLoadText.argtypes = [ctypes.c_char_p]
    try:
        assert l.HcclTuningTableLoadText(res.stdout.encode()) == 0
    finally:
        l.HcclTuningTableReset()


def test_packaged_tuning_table_is_well_formed():
    import ctypes

    from hccl_b200._lib import lib

    text = (ROOT / "hccl_b200" / "tuning" / "b200.txt").read_text()
    l = lib()
    l.HcclTuningTableLoadText.argtypes = [ctypes.c_char_p]
    try:
        assert l.HcclTuningTableLoadText(text.encode()) == 0
        names = ctypes.create_string_buffer(8192)
        for line in text.splitlines():
            if not line.strip() or line.startswith("#"):
                continue
            op, _, _, _, alg, _ = line.split()
            if alg == "none":
                continue
            opcode = {"allreduce": 2, "allgather": 6, "reducescatter": 7, "broadcast": 1, "alltoall": 10}[op]
            assert l.HcclListAlgorithms(opcode, names, 8192) == 0
            assert alg in names.value.decode().split(";"), f"{alg} is not a registered algorithm for {op}"
    finally:
        l.HcclTuningTableReset()


def test_checker_command_line(tmp_path, capsys):
    """python -m hccl_b200.utils.check: selector's choice, --all, a multi-level layout with a root, a count matrix, a text schedule with a
    lost notify (exit status 1) and the slice planner's cut."""
    from hccl_b200._lib import lib
    from hccl_b200.utils import check

    try:
        assert check.main(["--op", "allreduce", "--ranks", "4", "--count", "1000"]) == 0
        assert "ok: " in capsys.readouterr().out
        assert check.main(["--op", "scatter", "--ranks", "5", "--count", "77", "--root", "3", "--all"]) == 0
        out = capsys.readouterr().out
        assert "ok: InsScatterNHR" in out and "ok: SmScatterMesh1D" in out and "skipped: InsScatterSequenceMesh1DMesh1D" in out and "FAILED" not in out
        assert check.main(["--op", "broadcast", "--topo", "1x2x4", "--root", "5", "--count", "7001"]) == 0
        assert "InsBroadcastSequenceMesh1DMesh1D" in capsys.readouterr().out
        assert check.main(["--op", "alltoallv", "--ranks", "3", "--matrix", "1,0,7,300,1,0,4,5,6"]) == 0
        capsys.readouterr()
        # scratch far too small for the named algorithm's smallest chunk: reported, exit status 1
        assert check.main(["--op", "reduce", "--topo", "1x2x4", "--count", "1000", "--ccl-mb", "0.004"]) == 1
        assert "FAILED" in capsys.readouterr().out
        plan = tmp_path / "lost.txt"
        plan.write_text("op=BARRIER n=2 es=4 count=0 ccl=4096\nr0: POST 1 2; WAIT 1 2\nr1: WAIT 0 2\n")
        assert check.main(["--plan", str(plan)]) == 1
        assert "FAILED" in capsys.readouterr().out
        assert check.main(["--slices", "--op", "allgather", "--levels", "8@770,4@50", "--bytes", "67108864"]) == 0
        assert "modelled time" in capsys.readouterr().out
    finally:
        lib().HcclSetLogLevel(2)
