"""Worker for the lost-rank test: rank 1 leaves between operators without closing its communicator; rank 0 polls the
communicator status until the heartbeat reports the loss, then checks that the next operator is refused on the host."""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from hccl_b200._lib import HcclError  # noqa: E402
from hccl_b200.comm import init_from_env  # noqa: E402


def main():
    comm = init_from_env(backend="sim", buffer_mb=4)
    x = np.ones(128, np.float32)
    comm.all_reduce(x)
    comm.synchronize()
    comm.barrier()
    comm.synchronize()
    if comm.rank == 1:
        sys.stdout.flush()
        os._exit(0)                      # no destroy, no goodbye: the heartbeat connection just closes
    deadline = time.time() + 30
    while time.time() < deadline and comm.status() == 0:
        time.sleep(0.05)
    code = 0
    try:
        comm.all_reduce(x)
    except HcclError as e:
        code = e.code
    print(f"survivor saw status={comm.status()} code={code}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
