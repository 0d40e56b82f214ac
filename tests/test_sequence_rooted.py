"""Broadcast, Reduce and Scatter on two levels of the topology (the data crosses the servers once, through the root's column).

The generated plans go through the schedule checker (deadlock, scratch bounds, unordered accesses, symbolic result) for every
root of several layouts, whole and cut into chunks by a small scratch; then real data runs on the host simulation backend with
ranks laid out on pretended servers. Reference: src/ops/broadcast/executor/ins_v2_broadcast_sequence_executor.cc,
src/ops/reduce/executor/ins_v2_reduce_sequence_executor.cc, src/ops/scatter/executor/ins_v2_scatter_sequence_executor.cc."""
import ctypes

import numpy as np
import pytest

from hccl_b200._lib import lib
from hccl_b200.utils.sim import run_ranks

CMD = {"BROADCAST": 1, "REDUCE": 3, "SCATTER": 12}
ALG = {"BROADCAST": "InsBroadcastSequenceMesh1DMesh1D", "REDUCE": "InsReduceSequenceMesh1DMesh1D", "SCATTER": "InsScatterSequenceMesh1DMesh1D"}


def check(op, alg, topo, count, root, ccl=0):
    l = lib()
    buf = ctypes.create_string_buffer(1024)
    l.HcclCheckAlgorithm.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int,
                                     ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
    rc = l.HcclCheckAlgorithm(CMD[op], alg.encode(), topo[0], topo[1], topo[2], count, 4, root, None, ccl, buf, 1024)      # dtype 4 = fp32
    return rc, buf.value.decode()


@pytest.mark.parametrize("topo", [(1, 2, 2), (1, 2, 4), (1, 3, 2), (1, 4, 3)])
@pytest.mark.parametrize("op", ["BROADCAST", "REDUCE", "SCATTER"])
def test_plans_pass_the_schedule_checker_for_every_root(op, topo):
    n = topo[1] * topo[2]
    for root in range(n):
        for count in (1, 7, 1031) + ((20_000,) if root in (0, n - 1) else ()):
            rc, msg = check(op, ALG[op], topo, count, root)
            assert rc == 0, (root, count, msg)
            rc, msg = check(op, "", topo, count, root)                  # what the checker picks by itself on this layout
            assert rc == 0 and "Sequence" in msg, (root, count, msg)


@pytest.mark.parametrize("op", ["BROADCAST", "REDUCE", "SCATTER"])
def test_small_scratch_cuts_the_message_into_chunks(op):
    """96 KB of scratch for 200 KB per rank: several plans, each checked on its own, and together covering the message."""
    for root in (0, 5):
        rc, msg = check(op, ALG[op], (1, 2, 4), 50_001, root, ccl=96 << 10)
        assert rc == 0, (root, msg)


@pytest.mark.parametrize("op", ["BROADCAST", "REDUCE", "SCATTER"])
def test_scratch_too_small_for_any_chunk_is_an_error(op):
    rc, _ = check(op, ALG[op], (1, 2, 4), 1000, 0, ccl=8 << 10)
    assert rc != 0


@pytest.mark.parametrize("topo", ["1x2x2", "1x2x4", "1x3x2", "2x2x2"])
def test_rooted_operators_with_real_data(topo, monkeypatch):
    """The last layout has super-pods: everything above the server is folded into one level for these schedules."""
    pods, servers, per = (int(v) for v in topo.split("x"))
    n = pods * servers * per
    monkeypatch.setenv("HCCL_SIM_TOPO", topo)
    lib().HcclResetEnvConfigForTest()
    counts = (1, 5000, 200_003)
    roots = (0, n - 1, per)                      # first rank, last rank, first rank of the second server
    rng = np.random.default_rng(17)
    bc_in = {(c, r): rng.standard_normal(c).astype(np.float32) for c in counts for r in roots}
    rd_in = {c: [rng.integers(-8, 9, size=c).astype(np.float32) for _ in range(n)] for c in counts}
    sc_in = {(c, r): rng.standard_normal(c * n).astype(np.float32) for c in counts for r in roots}

    def body(comm, rank):
        out, algs = {}, set()
        for c in counts:
            for root in roots:
                b = bc_in[(c, root)].copy() if rank == root else np.zeros(c, np.float32)
                comm.broadcast(b, root)
                comm.synchronize()
                algs.add(comm.last_algorithm())
                red = np.full(c, -1.0, np.float32)
                comm.reduce(rd_in[c][rank], red, root)
                comm.synchronize()
                algs.add(comm.last_algorithm())
                sc = np.empty(c, np.float32)
                comm.scatter(sc_in[(c, root)] if rank == root else np.zeros(c * n, np.float32), sc, root)
                comm.synchronize()
                algs.add(comm.last_algorithm())
                out[(c, root)] = (b, red, sc)
        return out, algs

    try:
        res = run_ranks(n, body, buffer_mb=4)             # 2 MB per half: the largest count runs in chunks
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
    for rank, (out, algs) in enumerate(res):
        assert algs == set(ALG.values()), algs
        for c in counts:
            want_red = np.sum(np.stack(rd_in[c]).astype(np.float64), axis=0)
            for root in roots:
                b, red, sc = out[(c, root)]
                assert np.array_equal(b, bc_in[(c, root)]), (rank, c, root)
                if rank == root:
                    assert np.array_equal(red.astype(np.float64), want_red), (rank, c, root)
                else:
                    assert np.all(red == -1.0), (rank, c, root)          # only the root's receive buffer is written
                assert np.array_equal(sc, sc_in[(c, root)][rank * c:(rank + 1) * c]), (rank, c, root)


@pytest.mark.parametrize("op", ["BROADCAST", "REDUCE", "SCATTER"])
def test_super_pods_fold_into_the_upper_level_for_the_checker(op):
    for root in (0, 3, 7):
        rc, msg = check(op, "", (2, 2, 2), 1031, root)
        assert rc == 0 and "Sequence" in msg, (root, msg)


def test_all_gather_and_reduce_scatter_on_three_levels(monkeypatch):
    """AllGather and ReduceScatter are written for two levels; with super-pods they fold the upper two into one (AllReduce walks all three)."""
    n = 8
    monkeypatch.setenv("HCCL_SIM_TOPO", "2x2x2")
    lib().HcclResetEnvConfigForTest()
    rng = np.random.default_rng(3)
    c = 70_001
    ag_in = [rng.standard_normal(c).astype(np.float32) for _ in range(n)]
    rs_in = [rng.integers(-8, 9, size=c * n).astype(np.float32) for _ in range(n)]

    def body(comm, rank):
        g = np.empty(c * n, np.float32)
        comm.all_gather(ag_in[rank], g)
        comm.synchronize()
        a = comm.last_algorithm()
        s = np.empty(c, np.float32)
        comm.reduce_scatter(rs_in[rank], s)
        comm.synchronize()
        b = comm.last_algorithm()
        r = rs_in[rank][:c].copy()
        comm.all_reduce(r)
        comm.synchronize()
        return g, s, r, (a, b, comm.last_algorithm())

    try:
        res = run_ranks(n, body, buffer_mb=64)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
    want_rs = np.sum(np.stack(rs_in).astype(np.float64), axis=0)
    for rank, (g, s, r, algs) in enumerate(res):
        assert all("Sequence" in a for a in algs), algs
        assert np.array_equal(g, np.concatenate(ag_in))
        assert np.array_equal(s.astype(np.float64), want_rs[rank * c:(rank + 1) * c])
        assert np.array_equal(r.astype(np.float64), want_rs[:c])


def test_one_level_keeps_the_flat_algorithms(monkeypatch):
    """Without servers to cross nothing changes: the rooted operators keep their one-level algorithms."""
    lib().HcclResetEnvConfigForTest()

    def body(comm, rank):
        b = np.arange(100, dtype=np.float32) if rank == 1 else np.zeros(100, np.float32)
        comm.broadcast(b, 1)
        comm.synchronize()
        return b, comm.last_algorithm()

    for b, alg in run_ranks(4, body):
        assert np.array_equal(b, np.arange(100, dtype=np.float32))
        assert "Sequence" not in alg


def test_tree_forms_of_the_rooted_operators_with_real_data(monkeypatch):
    """HCCL_ALGO level1:NHR picks the tree scatter, the scatter + NHR all-gather broadcast and the NHR reduce-scatter + gather reduce
    (by name: InsScatterNHR, InsBroadcastNHR, ReduceNHR); odd rank count, every root, a message that runs in chunks."""
    n = 5
    monkeypatch.setenv("HCCL_ALGO", "level0:NA;level1:NHR")
    lib().HcclResetEnvConfigForTest()
    counts = (1, 7, 150_001)
    rng = np.random.default_rng(29)
    bc_in = {(c, r): rng.standard_normal(c).astype(np.float32) for c in counts for r in range(n)}
    rd_in = {c: [rng.integers(-8, 9, size=c).astype(np.float32) for _ in range(n)] for c in counts}
    sc_in = {(c, r): rng.standard_normal(c * n).astype(np.float32) for c in counts for r in range(n)}

    def body(comm, rank):
        out, algs = {}, set()
        for c in counts:
            for root in range(n):
                b = bc_in[(c, root)].copy() if rank == root else np.zeros(c, np.float32)
                comm.broadcast(b, root)
                comm.synchronize()
                algs.add(comm.last_algorithm())
                red = np.full(c, -1.0, np.float32)
                comm.reduce(rd_in[c][rank], red, root)
                comm.synchronize()
                algs.add(comm.last_algorithm())
                sc = np.empty(c, np.float32)
                comm.scatter(sc_in[(c, root)] if rank == root else np.zeros(c * n, np.float32), sc, root)
                comm.synchronize()
                algs.add(comm.last_algorithm())
                comm.barrier()
                comm.synchronize()
                algs.add(comm.last_algorithm())
                out[(c, root)] = (b, red, sc)
        return out, algs

    try:
        res = run_ranks(n, body, buffer_mb=2)             # 1 MB per half against 600 KB per rank (x 5 for the scatter)
    finally:
        monkeypatch.delenv("HCCL_ALGO")
        lib().HcclResetEnvConfigForTest()
    for rank, (out, algs) in enumerate(res):
        assert algs == {"InsBroadcastNHR", "ReduceNHR", "InsScatterNHR", "InsBarrierNHR"}, algs
        for c in counts:
            want_red = np.sum(np.stack(rd_in[c]).astype(np.float64), axis=0)
            for root in range(n):
                b, red, sc = out[(c, root)]
                assert np.array_equal(b, bc_in[(c, root)]), (rank, c, root)
                if rank == root:
                    assert np.array_equal(red.astype(np.float64), want_red), (rank, c, root)
                else:
                    assert np.all(red == -1.0), (rank, c, root)
                assert np.array_equal(sc, sc_in[(c, root)][rank * c:(rank + 1) * c]), (rank, c, root)


def test_two_level_barrier_orders_the_ranks(monkeypatch):
    """Nobody leaves the barrier before everybody has entered: each rank records its arrival in a shared list first."""
    import threading
    monkeypatch.setenv("HCCL_SIM_TOPO", "1x3x2")
    lib().HcclResetEnvConfigForTest()
    arrived, lock = [], threading.Lock()

    def body(comm, rank):
        seen = []
        for it in range(5):
            with lock:
                arrived.append((it, rank))
            comm.barrier()
            comm.synchronize()
            with lock:
                seen.append(sum(1 for i, _ in arrived if i == it))
        return seen, comm.last_algorithm()

    try:
        res = run_ranks(6, body)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
    for seen, alg in res:
        assert alg == "InsBarrierSequenceMesh1DMesh1D"
        assert seen == [6] * 5, seen


@pytest.mark.parametrize("topo", [(1, 2, 4), (1, 3, 2), (2, 2, 2)])
@pytest.mark.parametrize("op", ["BROADCAST", "REDUCE"])
def test_spread_forms_pass_the_schedule_checker(op, topo):
    """From 256 KB the message is cut into one slice per position of a server and every column carries its slice between the servers
    (Scatter always works that way); whole, and in chunks with 160 KB of scratch; a count that leaves the last slices short or empty."""
    n = topo[0] * topo[1] * topo[2]
    for root in (0, n - 1):
        for count, ccl in ((66_001, 0), (66_001, 160 << 10)):
            rc, msg = check(op, ALG[op], topo, count, root, ccl=ccl)
            assert rc == 0, (root, count, ccl, msg)


def test_reduce_sums_in_the_same_order_in_both_forms(monkeypatch):
    """The column form (small messages) and the spread form (from 256 KB) add the ranks of a server in rank order and then the servers in
    order: the first elements of a large Reduce carry the same bits as a small Reduce of just those elements."""
    topo, n = "1x2x4", 8
    monkeypatch.setenv("HCCL_SIM_TOPO", topo)
    lib().HcclResetEnvConfigForTest()
    rng = np.random.default_rng(31)
    full, few = 100_000, 1000
    xs = [(rng.standard_normal(full) * 10.0 ** rng.integers(-6, 6, full)).astype(np.float32) for _ in range(n)]

    def body(comm, rank):
        big = np.zeros(full, np.float32)
        comm.reduce(xs[rank], big, 5)
        comm.synchronize()
        small, head = np.zeros(few, np.float32), xs[rank][:few].copy()       # the operator is asynchronous: its input has to outlive the call
        comm.reduce(head, small, 5)
        comm.synchronize()
        return big, small

    try:
        res = run_ranks(n, body, buffer_mb=64)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
    big, small = res[5]
    assert np.array_equal(big[:few].view(np.uint32), small.view(np.uint32))
    servers = [np.zeros(full, np.float32) for _ in range(2)]
    for s in range(2):
        acc = xs[s * 4].copy()
        for r in range(1, 4):
            acc = acc + xs[s * 4 + r]
        servers[s] = acc
    assert np.array_equal(big.view(np.uint32), (servers[0] + servers[1]).view(np.uint32))


@pytest.mark.parametrize("groups, levels", [([[0, 1, 4, 5], [2, 3, 6, 7]], 2),        # two ranks of each server: still two regular servers
                                            ([[0, 4, 1, 5], [2, 6, 3, 7]], 1),        # servers interleaved in the rank order: one flat level
                                            ([[0, 1, 4], [2, 3, 5, 6, 7]], 1)])       # servers of unequal size: one flat level
def test_sub_communicators_keep_the_placement_of_their_ranks(groups, levels, monkeypatch):
    """A sub-communicator's ranks stay on the (pretended) servers they have in the parent. Where the picked ranks still form regular
    servers the multi-level executors serve it; any other layout runs the one-level algorithms, which are valid everywhere."""
    import ctypes as ct
    n, c = 8, 30_001
    monkeypatch.setenv("HCCL_SIM_TOPO", "1x2x4")
    lib().HcclResetEnvConfigForTest()
    xs = [np.random.default_rng(r).integers(-8, 9, size=c).astype(np.float32) for r in range(n)]

    def body(comm, rank):
        out = None
        for gi, g in enumerate(groups):
            sub = comm.create_sub_comm(g if rank in g else None, 100 + gi)
            if sub is None:
                continue
            desc = ct.create_string_buffer(2048)
            lib().HcclGetTopoDescription(ct.c_void_p(sub.handle), desc, 2048)
            a = xs[rank].copy()
            sub.all_reduce(a)
            sub.synchronize()
            algs = [sub.last_algorithm()]
            b = xs[g[1]].copy() if rank == g[1] else np.zeros(c, np.float32)
            sub.broadcast(b, 1)
            sub.synchronize()
            algs.append(sub.last_algorithm())
            gathered = np.empty(c * len(g), np.float32)
            sub.all_gather(xs[rank], gathered)
            sub.synchronize()
            algs.append(sub.last_algorithm())
            s = np.empty(c // len(g), np.float32)
            sub.reduce_scatter(xs[rank][:c // len(g) * len(g)], s)
            sub.synchronize()
            algs.append(sub.last_algorithm())
            out = (g, desc.value.decode(), algs, a, b, gathered, s)
            sub.destroy()
        return out

    try:
        res = run_ranks(n, body, buffer_mb=16)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
    for rank, (g, desc, algs, a, b, gathered, s) in enumerate(res):
        assert f"levels={levels}" in desc, desc
        assert all(("Sequence" in x or "Parallel" in x) == (levels == 2) for x in algs), algs
        total = np.sum(np.stack([xs[r] for r in g]).astype(np.float64), axis=0)
        assert np.array_equal(a.astype(np.float64), total)
        assert np.array_equal(b, xs[g[1]])
        assert np.array_equal(gathered, np.concatenate([xs[r] for r in g]))
        k, m = g.index(rank), c // len(g)
        assert np.array_equal(s.astype(np.float64), total[k * m:(k + 1) * m])


@pytest.mark.parametrize("seed", range(32))
def test_random_layouts_sizes_roots_and_scratch_sizes(seed, monkeypatch):
    """Six operators on a layout, message size, root, bandwidth weighting and scratch size drawn from the seed; whatever executor the
    selector picks (sequence, parallel, column or spread form, whole or in pieces) has to give the exact result."""
    import random
    rnd = random.Random(seed)
    topo = rnd.choice(["1x2x2", "1x2x3", "1x3x2", "1x2x4", "2x2x2", "1x4x2", "2x1x3", "3x1x2", "1x3x1", "2x2x1", "4x1x1"])
    bw = rnd.choice(["", "@2,1", "@1,2", "@0.5,0.5", "@5,1"])
    pods, servers, per = (int(v) for v in topo.split("x"))
    n = pods * servers * per
    buf = rnd.choice([1, 2, 4, 16])
    c = rnd.choice([1, 2, n - 1, n, n + 1, 1000, 4097, 65_537, 200_003, 500_009])
    cb = max(1, c // rnd.choice([1, 3, 7]))
    root = rnd.randrange(n)
    monkeypatch.setenv("HCCL_SIM_TOPO", topo + bw)
    lib().HcclResetEnvConfigForTest()
    rng = np.random.default_rng(seed)
    xs = [rng.integers(-8, 9, size=c).astype(np.float32) for _ in range(n)]
    blk = [rng.integers(-8, 9, size=cb).astype(np.float32) for _ in range(n)]
    blkn = [rng.integers(-8, 9, size=cb * n).astype(np.float32) for _ in range(n)]

    def body(comm, rank):
        a = xs[rank].copy()
        comm.all_reduce(a)
        g = np.empty(cb * n, np.float32)
        comm.all_gather(blk[rank], g)
        s = np.empty(cb, np.float32)
        comm.reduce_scatter(blkn[rank], s)
        b = xs[root].copy() if rank == root else np.zeros(c, np.float32)
        comm.broadcast(b, root)
        r = np.zeros(c, np.float32)
        comm.reduce(xs[rank], r, root)
        sc = np.zeros(cb, np.float32)
        comm.scatter(blkn[root], sc, root)
        comm.synchronize()
        return a, g, s, b, r, sc

    try:
        res = run_ranks(n, body, buffer_mb=buf)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
    total = np.sum(np.stack(xs).astype(np.float64), axis=0)
    total_blk = np.sum(np.stack(blkn).astype(np.float64), axis=0)
    what = (topo + bw, buf, c, cb, root)
    for rank, (a, g, s, b, r, sc) in enumerate(res):
        assert np.array_equal(a.astype(np.float64), total), what
        assert np.array_equal(g, np.concatenate(blk)), what
        assert np.array_equal(s.astype(np.float64), total_blk[rank * cb:(rank + 1) * cb]), what
        assert np.array_equal(b, xs[root]), what
        assert rank != root or np.array_equal(r.astype(np.float64), total), what
        assert np.array_equal(sc, blkn[root][rank * cb:(rank + 1) * cb]), what


def test_layout_description_of_another_size_is_ignored_with_a_warning_and_a_malformed_one_refused(monkeypatch):
    """HCCL_SIM_TOPO describes one communicator size; communicators of another size made beside it (a process group's sub-group, say)
    run on one pretended server. A value that is not <pods>x<servers>x<ranks> fails communicator creation."""
    from hccl_b200._lib import HcclError
    monkeypatch.setenv("HCCL_SIM_TOPO", "1x2x2")
    lib().HcclResetEnvConfigForTest()

    def body(comm, rank):
        x = np.full(10, rank + 1.0, np.float32)
        comm.all_reduce(x)
        comm.synchronize()
        return x[0], comm.last_algorithm()

    try:
        assert all(v == 6.0 and "Sequence" not in alg for v, alg in run_ranks(3, body))
        assert all(v == 10.0 and "Sequence" in alg for v, alg in run_ranks(4, body))
        monkeypatch.setenv("HCCL_SIM_TOPO", "banana")
        with pytest.raises(HcclError):
            run_ranks(2, body)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        lib().HcclResetEnvConfigForTest()
