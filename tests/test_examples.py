"""The samples are part of the product: they must build against the in-tree library and pass on the simulation backend;
on a multi-GPU machine the same binaries run on CUDA communicators."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples")
SAMPLES = ["comm_init_all", "send_recv", "batch_send_recv_ring", "allreduce", "broadcast", "allgather", "reduce_scatter", "reduce", "alltoall", "alltoallv",
           "alltoallvc", "scatter", "registered_allreduce", "custom_allgather"]


@pytest.fixture(scope="module")
def built():
    res = subprocess.run(["make", "-j8"], cwd=EX, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-4000:]
    return os.path.join(EX, "bin")


@pytest.mark.parametrize("name", SAMPLES)
@pytest.mark.parametrize("ranks", [2, 5])
def test_c_samples_on_simulation_backend(built, name, ranks):
    env = dict(os.environ, HCCL_BACKEND="sim", EXAMPLE_RANKS=str(ranks))
    res = subprocess.run([os.path.join(built, name)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0 and f"PASS: {ranks}/{ranks}" in res.stdout, res.stdout[-3000:]


def test_pytorch_backend_sample_on_cpu():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29561",
           os.path.join(EX, "pytorch", "allreduce_hccl_backend.py"), "--cpu"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0 and "hccl backend sample passed" in res.stdout, res.stdout[-4000:]


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("name", SAMPLES)
def test_c_samples_on_cuda(built, name):
    env = dict(os.environ, HCCL_DEVICE_WAIT_TIMEOUT_MS="10000")
    env.pop("HCCL_BACKEND", None)
    res = subprocess.run([os.path.join(built, name)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0 and "PASS" in res.stdout and "CUDA backend" in res.stdout, res.stdout[-3000:]
