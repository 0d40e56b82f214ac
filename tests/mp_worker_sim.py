"""Worker for the process-per-rank CPU test: init_from_env with the simulation backend under torchrun."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from hccl_b200.comm import init_from_env  # noqa: E402


def main():
    comm = init_from_env(backend="sim", buffer_mb=8)
    rank, world = comm.rank, comm.size
    x = np.full(10_000, rank + 1, dtype=np.float32)
    out = np.empty_like(x)
    comm.all_reduce(x, out)
    comm.synchronize()
    assert np.all(out == world * (world + 1) / 2), out[:4]
    g = np.empty(10_000 * world, dtype=np.float32)
    comm.all_gather(x, g)
    comm.synchronize()
    assert all(np.all(g[r * 10_000:(r + 1) * 10_000] == r + 1) for r in range(world))
    comm.barrier()
    comm.synchronize()
    comm.destroy()
    if rank == 0:
        print("sim process-per-rank ok", flush=True)


if __name__ == "__main__":
    main()
