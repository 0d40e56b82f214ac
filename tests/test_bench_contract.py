"""The parts of the benchmark contract that can be checked without a GPU."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_without_a_gpu_reports_unavailable_and_exits_zero():
    """On a GPU box the reference arm runs the unfused NCCL + cuBLAS baseline; without a device it must still exit 0 with
    the one-line reason, and it must never import this package."""
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]
    src = (ROOT / "bench.py").read_text()
    assert "from hccl_b200" in src and src.index("if ours:\n        sys.path.insert") < src.index("from hccl_b200._lib")


def test_graft_entry_exposes_build_and_smoke():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as g

    assert callable(g.build) and callable(g.smoke)


def test_public_headers_compile_as_c99(tmp_path):
    src = tmp_path / "hdr.c"
    src.write_text("".join(f'#include "hccl/{h}"\n' for h in ("hccl.h", "hccl_comm.h", "hccl_types.h", "hccl_mc2.h", "hccl_moe.h", "hccl_dfx.h",
                                                              "hccl_res.h", "hccl_graph_mode.h", "hccl_noalloc.h")) + "int main(void) { return 0; }\n")
    res = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{ROOT / 'include'}", "-c", str(src), "-o", str(tmp_path / "hdr.o")],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
