"""CPU-simulated plumbing test: 8 ranks, ring AllReduce (sum, fp32) on 1,048,576 elements per rank, inputs
N(0,1) with seed = rank, checked against an fp64 host sum at 1e-5 relative; then AllGather and ReduceScatter on the
same buffers."""
import numpy as np
import pytest

from hccl_b200.utils.sim import run_ranks

N_RANKS = 8
COUNT = 1 << 20


def _inputs():
    return [np.random.default_rng(r).standard_normal(COUNT).astype(np.float32) for r in range(N_RANKS)]


@pytest.mark.parametrize("algo", ["ring", "NHR", "fullmesh"])
def test_allreduce_allgather_reducescatter(monkeypatch, algo):
    monkeypatch.setenv("HCCL_ALGO", f"level0:NA;level1:{algo}")
    import ctypes
    from hccl_b200._lib import lib
    lib().HcclResetEnvConfigForTest()
    xs = _inputs()
    want = np.sum(np.stack(xs).astype(np.float64), axis=0)

    def body(comm, rank):
        x = xs[rank].copy()
        out = np.empty_like(x)
        comm.all_reduce(x, out)
        comm.synchronize()
        gathered = np.empty(COUNT // N_RANKS * N_RANKS, dtype=np.float32)
        comm.all_gather(x[: COUNT // N_RANKS], gathered)
        rs = np.empty(COUNT // N_RANKS, dtype=np.float32)
        comm.reduce_scatter(x, rs)
        comm.synchronize()
        return out, gathered, rs

    res = run_ranks(N_RANKS, body)
    denom = np.maximum(np.abs(want), 1.0)
    per = COUNT // N_RANKS
    for rank, (out, gathered, rs) in enumerate(res):
        assert np.max(np.abs(out - want) / denom) <= 1e-5
        assert np.array_equal(gathered, np.concatenate([x[:per] for x in xs]))
        assert np.max(np.abs(rs - want[rank * per:(rank + 1) * per]) / denom[rank * per:(rank + 1) * per]) <= 1e-5
    # every rank holds bit-identical all-reduce results
    for out, _, _ in res[1:]:
        assert np.array_equal(out, res[0][0])
    monkeypatch.delenv("HCCL_ALGO")
    lib().HcclResetEnvConfigForTest()
