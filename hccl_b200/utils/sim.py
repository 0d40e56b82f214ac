"""Rank-as-thread harness for the host simulation backend (no GPU needed).

`run_ranks(n, fn)` creates one communicator per rank, each on its own thread in this process, calls
`fn(comm, rank)` on every rank concurrently and returns the per-rank results; exceptions are re-raised in the
caller. This is the shape of HCCL's offline algorithm tests (one std::thread per rank), with real data.
"""
from __future__ import annotations

import threading
from typing import Callable, List

from ..comm import Communicator, get_root_info


def run_ranks(n: int, fn: Callable, *, buffer_mb: int = 0, timeout_s: float = 120.0, **comm_kw) -> List:
    root = get_root_info()
    results = [None] * n
    errors = [None] * n

    def body(rank: int):
        comm = None
        try:
            comm = Communicator.from_root_info(n, root, rank, buffer_mb=buffer_mb, backend="sim", **comm_kw)
            results[rank] = fn(comm, rank)
            comm.synchronize()
        except BaseException as e:  # noqa: BLE001
            errors[rank] = e
        finally:
            if comm is not None:
                try:
                    comm.destroy()
                except BaseException as e:  # noqa: BLE001
                    errors[rank] = errors[rank] or e

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    import time

    deadline = time.time() + timeout_s
    while time.time() < deadline and any(t.is_alive() for t in threads):
        # a rank that raised leaves its peers waiting inside a collective: report the error, not the wait
        if any(e is not None for e in errors):
            grace = time.time() + 2.0
            while time.time() < grace and any(t.is_alive() for t in threads):
                time.sleep(0.02)
            break
        time.sleep(0.02)
    for e in errors:
        if e is not None:
            raise e
    if any(t.is_alive() for t in threads):
        raise TimeoutError("a simulated rank did not finish")
    return results
