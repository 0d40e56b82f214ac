"""Process-per-rank on CPU: ranks are separate processes started by torchrun, the heap is shared memory passed as file
descriptors over unix sockets, the root info travels through a TCPStore."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_two_processes_sim_backend():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(HERE, "mp_worker_sim.py")]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "sim process-per-rank ok" in res.stdout


def test_four_processes_on_two_pretended_servers():
    """The same worker with ranks laid out on two servers of two: the multi-level executors run between processes as well."""
    env = dict(os.environ, HCCL_SIM_TOPO="1x2x2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1", "--master-port", "29535",
           os.path.join(HERE, "mp_worker_sim.py")]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "sim process-per-rank ok" in res.stdout
    assert "levels=2" in res.stdout, res.stdout[-2000:]
