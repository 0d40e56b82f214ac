"""torch.distributed backend "hccl": on CPU (host simulation backend, 2 processes) and, when GPUs exist, on CUDA."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _ensure_ext():
    from hccl_b200.parallel import process_group
    if not process_group.EXT_PATH.exists():
        from hccl_b200.utils import build
        build.build_torch_ext()


def _run(nproc, device, port):
    _ensure_ext()
    env = dict(os.environ, PG_DEVICE=device)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "mp_worker_pg.py")]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-6000:]
    assert "process group checks passed" in res.stdout


def test_process_group_cpu_two_ranks():
    _run(2, "cpu", 29581)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_process_group_cuda():
    _run(min(torch.cuda.device_count(), 8), "cuda", 29583)
