"""Every public operator on the host simulation backend (ranks are threads, data really moves), against numpy oracles.

The sweep follows the reference's operator test matrix (test/st/algorithm/testcase/testcase_all_reduce.cpp and the
sibling testcase_*.cpp files: op x data type x reduce op x rank count x boundary sizes), with real payloads instead of
symbolic ones.
"""
import ctypes

import numpy as np
import pytest
import torch

from hccl_b200._lib import HcclError, lib
from hccl_b200.types import ReduceOp, Result
from hccl_b200.utils.sim import run_ranks

NP_DTYPES = [np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64, np.float16, np.float32, np.float64]
REDUCE = {ReduceOp.SUM: np.add, ReduceOp.PROD: np.multiply, ReduceOp.MAX: np.maximum, ReduceOp.MIN: np.minimum}


def make(rank, count, dtype, salt=0):
    rng = np.random.default_rng(1000 * salt + rank)
    if np.issubdtype(dtype, np.integer):
        return rng.integers(1, 4, size=count).astype(dtype)   # small values: sums and products of 8 stay exact in int8
    return (rng.integers(-8, 9, size=count) / 4.0).astype(dtype)


def oracle_reduce(xs, op):
    acc = xs[0].copy()
    for x in xs[1:]:
        acc = REDUCE[op](acc, x)
    return acc


@pytest.mark.parametrize("nranks", [2, 3, 5, 8])
@pytest.mark.parametrize("dtype", NP_DTYPES, ids=lambda d: np.dtype(d).name)
def test_allreduce_dtypes_and_ops(nranks, dtype):
    counts = [1, nranks + 1, 1000]
    ops = list(REDUCE)
    xs = {(c, o): [make(r, c, dtype, salt=c + int(o)) for r in range(nranks)] for c in counts for o in ops}

    def body(comm, rank):
        outs = {}
        for key, inputs in xs.items():
            out = np.empty_like(inputs[rank])
            comm.all_reduce(inputs[rank], out, op=key[1])      # calls are asynchronous: buffers stay alive until synchronize()
            outs[key] = out
        comm.synchronize()
        return outs

    res = run_ranks(nranks, body)
    for key, inputs in xs.items():
        if key[1] == ReduceOp.PROD and np.issubdtype(dtype, np.floating):
            inputs64 = [x.astype(np.float64) for x in inputs]
            want = oracle_reduce(inputs64, key[1])
            for r in range(nranks):
                assert np.allclose(res[r][key].astype(np.float64), want, rtol=2e-2 if dtype == np.float16 else 1e-6), key
            continue
        want = oracle_reduce(inputs, key[1])
        for r in range(nranks):
            assert np.array_equal(res[r][key], want), (key, r)


@pytest.mark.parametrize("nranks", [2, 4, 7])
def test_bf16_through_torch_cpu_tensors(nranks):
    xs = [torch.randint(-8, 9, (515,), generator=torch.Generator().manual_seed(r)).to(torch.bfloat16) / 4 for r in range(nranks)]
    want = torch.stack([x.float() for x in xs]).sum(0)

    def body(comm, rank):
        out = torch.empty_like(xs[rank])
        comm.all_reduce(xs[rank], out)
        g = torch.empty(nranks * 515, dtype=torch.bfloat16)
        comm.all_gather(xs[rank], g)
        comm.synchronize()
        return out, g

    for out, g in run_ranks(nranks, body):
        assert torch.equal(out.float(), want)
        assert torch.equal(g, torch.cat(xs))


@pytest.mark.parametrize("nranks", [2, 3, 4, 8])
def test_rooted_and_gather_scatter_ops(nranks):
    count = 777
    dtype = np.float32
    xs = [make(r, count, dtype) for r in range(nranks)]
    big = [make(r, count * nranks, dtype, salt=7) for r in range(nranks)]

    def body(comm, rank):
        out = {}
        for root in (0, nranks - 1):
            b = xs[root].copy() if rank == root else np.zeros(count, dtype)
            comm.broadcast(b, root)
            out["bcast", root] = b
            red = np.full(count, -1, dtype)
            comm.reduce(xs[rank], red, root, op=ReduceOp.MAX)
            out["reduce", root] = red
            sc = np.empty(count, dtype)
            comm.scatter(big[root] if rank == root else None, sc, root)
            out["scatter", root] = sc
        ag = np.empty(count * nranks, dtype)
        comm.all_gather(xs[rank], ag)
        out["ag"] = ag
        rs = np.empty(count, dtype)
        comm.reduce_scatter(big[rank], rs)
        out["rs"] = rs
        a2a = np.empty(count * nranks, dtype)
        comm.all_to_all(big[rank], a2a)
        out["a2a"] = a2a
        comm.barrier()
        comm.synchronize()
        return out

    res = run_ranks(nranks, body)
    rs_want = oracle_reduce(big, ReduceOp.SUM)
    for r, out in enumerate(res):
        for root in (0, nranks - 1):
            assert np.array_equal(out["bcast", root], xs[root])
            if r == root:
                assert np.array_equal(out["reduce", root], oracle_reduce(xs, ReduceOp.MAX))
            else:
                assert np.all(out["reduce", root] == -1)   # non-root outputs untouched
            assert np.array_equal(out["scatter", root], big[root][r * count:(r + 1) * count])
        assert np.array_equal(out["ag"], np.concatenate(xs))
        assert np.array_equal(out["rs"], rs_want[r * count:(r + 1) * count])
        assert np.array_equal(out["a2a"], np.concatenate([big[s][r * count:(r + 1) * count] for s in range(nranks)]))


@pytest.mark.parametrize("nranks", [2, 3, 5, 8])
def test_variable_count_ops(nranks):
    dtype = np.int32
    M = [[((3 * i + 5 * j) % 4) * 11 + (1 if (i + j) % 3 == 0 else 0) for j in range(nranks)] for i in range(nranks)]
    send = [np.arange(sum(M[r]), dtype=dtype) + 10000 * r for r in range(nranks)]
    vcnt = [(7 * r) % 5 * 13 for r in range(nranks)]      # includes zero-length contributions
    vdis = list(np.cumsum([0] + vcnt[:-1]))
    vsrc = [make(r, vcnt[r], dtype, salt=3) for r in range(nranks)]
    rsv_in = [make(r, sum(vcnt), dtype, salt=4) for r in range(nranks)]

    def body(comm, rank):
        sc = M[rank]
        sd = list(np.cumsum([0] + sc[:-1]))
        rc = [M[s][rank] for s in range(nranks)]
        rd = list(np.cumsum([0] + rc[:-1]))
        o1 = np.full(max(1, sum(rc)), -1, dtype)
        comm.all_to_all_v(send[rank], sc, sd, o1, rc, rd)
        o2 = np.full(max(1, sum(rc)), -1, dtype)
        comm.all_to_all_vc(send[rank], M, o2)
        o3 = np.full(sum(vcnt), -1, dtype)
        comm.all_gather_v(vsrc[rank] if vcnt[rank] else None, o3, vcnt, vdis)
        o4 = np.full(max(1, vcnt[rank]), -1, dtype)
        comm.reduce_scatter_v(rsv_in[rank], vcnt, vdis, o4 if vcnt[rank] else None)
        comm.synchronize()
        return o1[:sum(rc)], o2[:sum(rc)], o3, o4[:vcnt[rank]]

    res = run_ranks(nranks, body)
    rsv_want = oracle_reduce(rsv_in, ReduceOp.SUM)
    for r, (o1, o2, o3, o4) in enumerate(res):
        pieces = []
        for s in range(nranks):
            off = sum(M[s][:r])
            pieces.append(send[s][off:off + M[s][r]])
        want = np.concatenate(pieces) if pieces else np.empty(0, dtype)
        assert np.array_equal(o1, want)
        assert np.array_equal(o2, want)
        assert np.array_equal(o3, np.concatenate(vsrc))
        assert np.array_equal(o4, rsv_want[vdis[r]:vdis[r] + vcnt[r]])


@pytest.mark.parametrize("nranks", [3, 4])
def test_alltoallv_zero_row_zero_column_and_pairs_above_the_scratch_half(nranks):
    """A rank that sends nothing, a rank that receives nothing, and pairs larger than half of a 1 MB scratch window."""
    dtype = np.int32
    M = [[4000 * ((i + 2 * j) % 3) + 7 * (i + 1) for j in range(nranks)] for i in range(nranks)]
    M[0][nranks - 1] = 160_000                         # 640 KB in one pair
    M[nranks - 1][0] = 1
    for j in range(nranks):
        M[1][j] = 0
        M[j][2] = 0
    send = [np.arange(max(1, sum(M[r])), dtype=dtype) + 1_000_000 * r for r in range(nranks)]

    def body(comm, rank):
        sc = M[rank]
        sd = list(np.cumsum([0] + sc[:-1]))
        rc = [M[s][rank] for s in range(nranks)]
        rd = list(np.cumsum([0] + rc[:-1]))
        o1 = np.full(max(1, sum(rc)), -1, dtype)
        comm.all_to_all_v(send[rank], sc, sd, o1, rc, rd)
        o2 = np.full(max(1, sum(rc)), -1, dtype)
        comm.all_to_all_vc(send[rank], M, o2)
        comm.synchronize()
        return o1, o2, sum(rc)

    res = run_ranks(nranks, body, buffer_mb=1)
    for r, (o1, o2, total) in enumerate(res):
        pieces = [send[s][sum(M[s][:r]):sum(M[s][:r]) + M[s][r]] for s in range(nranks)]
        want = np.concatenate(pieces)
        assert want.size == total
        assert np.array_equal(o1[:total], want) and np.array_equal(o2[:total], want)
        assert np.all(o1[total:] == -1) and np.all(o2[total:] == -1)


@pytest.mark.parametrize("nranks", [2, 4, 5])
def test_point_to_point_and_batch(nranks):
    count = 3001

    def body(comm, rank):
        nxt, prv = (rank + 1) % nranks, (rank - 1) % nranks
        mine = np.full(count, rank, np.int64)
        got = np.empty(count, np.int64)
        # even ranks send first, odd ranks receive first (a ring of blocking pairs must not deadlock)
        if rank % 2 == 0:
            comm.send(mine, nxt)
            comm.recv(got, prv)
        else:
            comm.recv(got, prv)
            comm.send(mine, nxt)
        comm.synchronize()
        got2a, got2b = np.empty(count, np.int64), np.empty(17, np.int64)
        back = mine[:17] + 100
        comm.batch_send_recv([("send", mine, nxt), ("recv", got2a, prv), ("send", back, prv), ("recv", got2b, nxt)])
        comm.synchronize()
        return got, got2a, got2b

    if nranks % 2 == 1:
        # with an odd ring the "even sends first" rule pairs two senders (last and first): use the batch form only
        def body(comm, rank):   # noqa: F811
            nxt, prv = (rank + 1) % nranks, (rank - 1) % nranks
            mine = np.full(count, rank, np.int64)
            got, got2a, got2b = np.empty(count, np.int64), np.empty(count, np.int64), np.empty(17, np.int64)
            back = mine[:17] + 100
            comm.batch_send_recv([("send", mine, nxt), ("recv", got, prv)])
            comm.batch_send_recv([("send", mine, nxt), ("recv", got2a, prv), ("send", back, prv), ("recv", got2b, nxt)])
            comm.synchronize()
            return got, got2a, got2b

    for r, (got, a, b) in enumerate(run_ranks(nranks, body)):
        prv, nxt = (r - 1) % nranks, (r + 1) % nranks
        assert np.all(got == prv) and np.all(a == prv) and np.all(b == nxt + 100)


def test_large_payload_goes_through_the_chunk_loop():
    nranks, count = 4, 3 * (1 << 20) // 4 + 13          # 3 MB + tail through a 1 MB scratch window
    xs = [make(r, count, np.float32) for r in range(nranks)]

    def body(comm, rank):
        out = np.empty_like(xs[rank])
        comm.all_reduce(xs[rank], out)
        ag = np.empty(count * nranks, np.float32)
        comm.all_gather(xs[rank], ag)
        b = xs[2].copy() if rank == 2 else np.zeros(count, np.float32)
        comm.broadcast(b, 2)
        comm.synchronize()
        c = (ctypes.c_uint64 * 9)()
        lib().HcclGetCommCounters(ctypes.c_void_p(comm.handle), c)
        return out, ag, b, c[7]

    res = run_ranks(nranks, body, buffer_mb=1)
    want = oracle_reduce(xs, ReduceOp.SUM)
    for out, ag, b, loops in res:
        assert np.array_equal(out, want)
        assert np.array_equal(ag, np.concatenate(xs))
        assert np.array_equal(b, xs[2])
        assert loops >= 3


def test_in_place_and_zero_count():
    nranks = 4
    xs = [make(r, 100, np.float32) for r in range(nranks)]

    def body(comm, rank):
        x = xs[rank].copy()
        comm.all_reduce(x)                                 # send == recv
        empty = np.empty(0, np.float32)
        comm.all_reduce(empty, empty)                      # count 0: a no-op that still returns success
        comm.synchronize()
        return x

    want = oracle_reduce(xs, ReduceOp.SUM)
    for x in run_ranks(nranks, body):
        assert np.array_equal(x, want)


def test_parameter_errors_are_reported_not_crashes():
    def body(comm, rank):
        codes = []
        x = np.zeros(8, np.float32)
        for call in (lambda: comm.broadcast(x, 99),                                # root out of range
                     lambda: comm.send(x, comm.size + 3),                          # peer out of range
                     lambda: comm.send(x, rank),                                   # self send
                     lambda: comm.reduce(x, x.copy(), 0, op=7)):                   # bad reduce op
            try:
                call()
                codes.append(0)
            except HcclError as e:
                codes.append(e.code)
        h = ctypes.c_void_p(comm.handle)
        codes.append(lib().HcclAllReduce(None, None, 8, 4, 0, h, None))            # null buffers
        codes.append(lib().HcclAllReduce(x.ctypes.data, x.ctypes.data, 8, 99, 0, h, None))  # bad dtype
        codes.append(lib().HcclAllReduce(x.ctypes.data, x.ctypes.data, 8, 15, 0, h, None))  # fp8 has no reduction
        codes.append(lib().HcclAllReduce(x.ctypes.data, x.ctypes.data, 8, 4, 0, None, None))  # null comm
        # the communicator is still usable afterwards
        comm.all_reduce(x)
        comm.synchronize()
        return codes

    for codes in run_ranks(2, body):
        assert codes[0] == Result.E_PARA and codes[1] == Result.E_PARA and codes[2] == Result.E_PARA and codes[3] == Result.E_PARA
        assert codes[4] == Result.E_PTR
        assert codes[5] in (Result.E_PARA, Result.E_NOT_SUPPORT)
        assert codes[6] in (Result.E_PARA, Result.E_NOT_SUPPORT)
        assert codes[7] == Result.E_PTR


@pytest.mark.parametrize("algo", ["fullmesh"])
def test_reductions_are_batch_invariant(monkeypatch, algo):
    """The value of an element does not depend on how many other elements travel with it or on the scratch size (chunking):
    mesh reductions add in rank order whatever the count. This is the property the reference's experimental batch-invariant
    ReduceScatter adds for its 2-D topology (docs/en/rfcs/0001-add-batch-invariant-reducescatter.md)."""
    monkeypatch.setenv("HCCL_ALGO", f"level0:NA;level1:{algo}")
    lib().HcclResetEnvConfigForTest()
    nranks, n = 5, 40_000
    rng = np.random.default_rng(7)
    xs = [(rng.standard_normal(n) * 10.0 ** rng.integers(-6, 6, n)).astype(np.float32) for _ in range(nranks)]

    def run(count, buffer_mb):
        def body(comm, rank):
            out = np.empty(count, np.float32)
            comm.all_reduce(xs[rank][:count], out)
            blk = count // nranks
            rs = np.empty(blk, np.float32)
            comm.reduce_scatter(xs[rank][:blk * nranks], rs)
            comm.synchronize()
            return out, rs
        return run_ranks(nranks, body, buffer_mb=buffer_mb)

    try:
        full = run(n, 0)
        small = run(n // 7, 0)
        chunked = run(n, 1)                      # 1 MB scratch is plenty here; still a different plan geometry
        for r in range(nranks):
            assert np.array_equal(full[r][0][: n // 7].view(np.uint32), small[r][0].view(np.uint32))
            assert np.array_equal(full[r][0].view(np.uint32), chunked[r][0].view(np.uint32))
            assert np.array_equal(full[r][0].view(np.uint32), full[0][0].view(np.uint32))      # and identical on every rank
    finally:
        monkeypatch.delenv("HCCL_ALGO")
        lib().HcclResetEnvConfigForTest()
