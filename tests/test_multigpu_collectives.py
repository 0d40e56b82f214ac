"""Real multi-GPU runs of the C API (one process per GPU over NVLink): every operator, several dtypes, chunk loops forced by
a small CCL buffer, with the NVLS engine on and off."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, extra_env, port, worker="mp_worker_collectives.py", expect="all multi-GPU collective checks passed"):
    env = dict(os.environ)
    env.update(extra_env)
    env.setdefault("HCCL_DEVICE_WAIT_TIMEOUT_MS", "10000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, worker)]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-6000:]
    assert expect in res.stdout, res.stdout[-3000:]


@pytest.mark.parametrize("cfg", [
    {"HCCL_NVLS_ENABLE": "0"},
    {"HCCL_NVLS_ENABLE": "0", "HCCL_BUFFSIZE": "4"},
    {"HCCL_NVLS_ENABLE": "1"},
    {"HCCL_NVLS_ENABLE": "1", "HCCL_BUFFSIZE": "4"},
    {"HCCL_NVLS_ENABLE": "0", "HCCL_OP_EXPANSION_MODE": "COPY_ENGINE", "HCCL_BUFFSIZE": "16"},
    {"HCCL_NVLS_ENABLE": "1", "HCCL_BUFFSIZE": "8", "HCCL_ALGO_NAME": "allreduce=NvlsAllReducePipelined;allgather=NvlsAllGatherPush;"
     "reducescatter=NvlsReduceScatterPipelined;allgatherv=NvlsAllGatherVPush;reducescatterv=SmReduceScatterVPipelined;"
     "broadcast=NvlsBroadcastPush;alltoall=SmAlltoAllPush"},
    {"HCCL_NVLS_ENABLE": "0", "HCCL_BUFFSIZE": "8", "HCCL_ALGO_NAME": "allreduce=SmAllReducePipelined;allgather=SmAllGatherPush;"
     "reducescatter=SmReduceScatterPipelined;allgatherv=SmAllGatherVPush;reducescatterv=SmReduceScatterVPipelined;"
     "broadcast=SmBroadcastPush;alltoall=SmAlltoAllPush"},
])
def test_collectives_two_or_more_gpus(cfg):
    n = min(torch.cuda.device_count(), 8)
    _run(n, cfg, 29610 + len(cfg) * 7 + int(cfg.get("HCCL_NVLS_ENABLE", "0")) * 3 + len(cfg.get("HCCL_OP_EXPANSION_MODE", "")) + len(cfg.get("HCCL_ALGO_NAME", "")) % 97)


def test_fused_matmul_collectives_two_or_more_gpus():
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    _run(n, {}, 29655, worker="mp_worker_fused.py", expect="all fused multi-GPU checks passed")


def test_data_parallel_two_or_more_gpus():
    """Bucketed gradient all-reduce on real GPUs: registered buckets (zero-copy, in place) and ordinary buckets (staged)."""
    n = min(torch.cuda.device_count(), 4)
    _run(n, {}, 29671, worker="mp_worker_dp.py", expect="data-parallel checks passed")
