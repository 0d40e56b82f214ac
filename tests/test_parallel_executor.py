"""The Parallel executors (two levels of the topology busy at once) and their slice planner.

Three layers of evidence: the planner's arithmetic, the schedule checker over the generated plans (deadlock, scratch bounds,
unordered accesses between the queues and ranks, symbolic result), and real data on the host simulation backend with ranks
laid out on pretended servers. Reference: the OmniPipe slice calculation and the Parallel executors
(src/ops/op_common/omnipipe_data_slice_calc.cc, src/ops/all_reduce/executor/ins_v2_all_reduce_parallel_executor.cc)."""
import ctypes

import numpy as np
import pytest

from hccl_b200._lib import lib
from hccl_b200.types import ReduceOp
from hccl_b200.utils.sim import run_ranks

CMD = {"ALLREDUCE": 2, "ALLGATHER": 6, "REDUCE_SCATTER": 7}


def _cmd(name):
    return CMD[name]


def plan(op, n0, bw0, n1, bw1, nbytes):
    l = lib()
    l.HcclPlanParallelSlices.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_double, ctypes.c_uint32, ctypes.c_double, ctypes.c_uint64,
                                         ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_double),
                                         ctypes.POINTER(ctypes.c_double)]
    sb, ss = (ctypes.c_uint64 * 2)(), (ctypes.c_uint32 * 2)()
    seq, par = ctypes.c_double(), ctypes.c_double()
    rc = l.HcclPlanParallelSlices(_cmd(op), n0, bw0, n1, bw1, nbytes, sb, ss, ctypes.byref(seq), ctypes.byref(par))
    assert rc == 0
    return list(sb), list(ss), seq.value, par.value


def check(op, alg, topo, count, ccl=0):
    l = lib()
    buf = ctypes.create_string_buffer(1024)
    l.HcclCheckAlgorithm.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int,
                                     ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
    rc = l.HcclCheckAlgorithm(_cmd(op), alg.encode(), topo[0], topo[1], topo[2], count, 4, 0, None, ccl, buf, 1024)      # dtype 4 = fp32
    return rc, buf.value.decode()


# ---------------------------------------------------------------------------------------------------------------- planner
@pytest.mark.parametrize("op", ["ALLGATHER", "REDUCE_SCATTER", "ALLREDUCE"])
def test_planner_shares_cover_the_block_are_aligned_and_balance_the_levels(op):
    nbytes = 64 << 20
    shares, steps, seq, par = plan(op, 4, 200.0, 4, 100.0, nbytes)
    assert sum(shares) == nbytes and all(b % 512 == 0 for b in shares)
    assert shares[0] > 0 and shares[1] > 0 and all(1 <= s <= 4 for s in steps)
    assert par < seq                                     # both levels busy beats one after the other
    if op == "ALLGATHER":
        # loads cross where 3 (4 - 3a) / 200 = 3 (1 + 3a) / 100: two ninths of the block start inside the server
        assert abs(shares[0] / nbytes - 2 / 9) < 1e-3


def test_planner_keeps_one_share_when_one_level_is_the_bottleneck_either_way():
    """NVLink inside the server against a network 15 times slower: sending a block over the network once (first) beats every
    mix, so there is one share; its steps still overlap the two levels."""
    nbytes = 64 << 20
    shares, steps, seq, par = plan("ALLGATHER", 8, 770.0, 4, 50.0, nbytes)
    assert shares == [0, nbytes] and steps[1] == 4
    assert par < 0.8 * seq


def test_planner_follows_the_bandwidth_ratio():
    nbytes = 32 << 20
    a = plan("ALLGATHER", 4, 400.0, 4, 400.0, nbytes)[0]
    b = plan("ALLGATHER", 4, 400.0, 4, 40.0, nbytes)[0]
    assert abs(a[0] - a[1]) <= 1024                      # a symmetric grid is cut in the middle
    assert b[1] > a[1]                                   # a slower level 1 sends more of the block through it FIRST (1 block instead of 4)


def test_planner_degenerate_cases_keep_one_share():
    for n0, n1 in ((1, 8), (8, 1)):
        shares, steps, seq, par = plan("ALLREDUCE", n0, 770.0, n1, 50.0, 1 << 20)
        assert sorted(shares) == [0, 1 << 20] and par == seq
    shares, _, _, _ = plan("ALLGATHER", 4, 770.0, 2, 50.0, 600)      # less than two aligned pieces
    assert sorted(shares) == [0, 600]


def test_planner_invariants_over_random_grids():
    """Whatever the grid, the bandwidths and the size: the shares cover the block exactly, a cut between two shares is aligned, step counts
    stay within bounds, the priced times are positive, and a faster level 1 never shrinks the share that leans on it (the one that starts inside the server and then
    forwards the server's blocks over level 1)."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=300, deadline=None)
    @given(st.sampled_from(["ALLGATHER", "REDUCE_SCATTER", "ALLREDUCE"]), st.integers(1, 16), st.floats(1.0, 1000.0), st.integers(1, 16),
           st.floats(1.0, 1000.0), st.integers(1, 1 << 30))
    def prop(op, n0, bw0, n1, bw1, nbytes):
        shares, steps, seq, par = plan(op, n0, bw0, n1, bw1, nbytes)
        assert sum(shares) == nbytes
        assert seq > 0 and par > 0
        if shares[0] and shares[1]:
            assert shares[0] % 512 == 0                      # the cut; the second share takes the (possibly unaligned) rest
        for b, k in zip(shares, steps):
            assert (b == 0) == (k == 0) and k <= 4
        faster = plan(op, n0, bw0, n1, bw1 * 4.0, nbytes)[0]
        if op == "ALLGATHER":
            assert faster[0] >= shares[0] - 512

    prop()


# ---------------------------------------------------------------------------------------------------------------- checker
@pytest.mark.parametrize("topo", [(1, 2, 2), (1, 2, 4), (1, 3, 2), (1, 4, 2), (1, 2, 8), (2, 2, 2)])
@pytest.mark.parametrize("op", ["ALLGATHER", "REDUCE_SCATTER", "ALLREDUCE"])
def test_parallel_plans_pass_the_schedule_checker(op, topo):
    alg = {"ALLGATHER": "InsAllGatherParallelMesh1DMesh1D", "REDUCE_SCATTER": "InsReduceScatterParallelMesh1DMesh1D", "ALLREDUCE": "InsAllReduceParallelMesh1DMesh1D"}[op]
    big = 70_001 if topo[1] * topo[2] <= 8 else 40_001  # the checker tracks every element: keep the 16-rank case short
    for count in (1, 1000, big):                        # one share only, two shares of one step, several steps with an odd tail
        rc, msg = check(op, alg, topo, count, ccl=64 << 20)
        assert rc == 0, (count, msg)


def test_parallel_plans_over_random_layouts_and_counts():
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=40, deadline=None)
    @given(st.sampled_from(["ALLGATHER", "REDUCE_SCATTER", "ALLREDUCE"]), st.integers(2, 4), st.integers(2, 4), st.integers(1, 50_000))
    def prop(op, servers, per, count):
        alg = {"ALLGATHER": "InsAllGatherParallelMesh1DMesh1D", "REDUCE_SCATTER": "InsReduceScatterParallelMesh1DMesh1D", "ALLREDUCE": "InsAllReduceParallelMesh1DMesh1D"}[op]
        rc, msg = check(op, alg, (1, servers, per), count, ccl=64 << 20)
        assert rc == 0, (op, servers, per, count, msg)

    prop()


def test_parallel_plan_reports_a_scratch_window_that_is_too_small():
    """A call larger than the scratch is cut into pieces; a scratch that cannot hold a piece of 1024 elements is reported."""
    rc, msg = check("ALLGATHER", "InsAllGatherParallelMesh1DMesh1D", (1, 2, 4), 100_000, ccl=1 << 20)
    assert rc == 0, msg
    rc, msg = check("ALLGATHER", "InsAllGatherParallelMesh1DMesh1D", (1, 2, 4), 100_000, ccl=2 << 10)
    assert rc != 0


def test_checker_orders_queues_of_one_rank_by_their_local_notifies():
    l = lib()
    l.HcclCheckPlanText.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32]
    buf = ctypes.create_string_buffer(512)
    good = """op=6 n=2 es=4 count=4 ccl=4096
r0: COPY ccl@0 in@0 16; LPOST 1
r0.q1: LWAIT 0; POST 1 3; WAIT 1 3; READ 1 out@16 ccl@0 16; COPY out@0 in@0 16
r1: COPY ccl@0 in@0 16; LPOST 1
r1.q1: LWAIT 0; POST 0 3; WAIT 0 3; READ 0 out@0 ccl@0 16; COPY out@16 in@0 16
"""
    assert l.HcclCheckPlanText(good.encode(), buf, 512) == 0, buf.value
    racy = good.replace("LWAIT 0; ", "").replace("; LPOST 1", "")          # queue 1 no longer waits for the staging copy of queue 0
    assert l.HcclCheckPlanText(racy.encode(), buf, 512) != 0
    assert b"not ordered" in buf.value
    lost = good.replace("r0.q1: LWAIT 0; ", "r0.q1: ")                     # a local notify nobody waits for
    assert l.HcclCheckPlanText(lost.encode(), buf, 512) != 0


# ---------------------------------------------------------------------------------------------------------------- real data
def _oracle(xs):
    acc = xs[0].astype(np.float64)
    for x in xs[1:]:
        acc = acc + x
    return acc


@pytest.mark.parametrize("topo", ["1x2x2", "1x2x4@2,1", "1x3x2@0.8,0.6", "2x2x2@2,1,1"])
@pytest.mark.parametrize("forced", [True, False], ids=["by-name", "selected"])
def test_two_level_operators_with_real_data(topo, forced, monkeypatch):
    """Ranks as threads on pretended servers; the same calls once with the parallel executors named and once left to the selector,
    which has to follow the planner: the parallel form where it is priced a tenth below the sequential one, else the sequence
    executors. The bandwidth weights after '@' (GB/s) make the two levels comparable and slow enough that 1.2 MB is bandwidth-bound in the model."""
    pods, servers, per = (int(v) for v in topo.split("@")[0].split("x"))
    bw = [float(v) for v in topo.split("@")[1].split(",")] if "@" in topo else None
    n = pods * servers * per
    servers *= pods                      # super-pods fold into the upper level: every server of every pod
    if bw and len(bw) == 3:
        bw = [bw[0], min(bw[1:])]
    monkeypatch.setenv("HCCL_SIM_TOPO", topo)
    if forced:
        monkeypatch.setenv("HCCL_ALGO_NAME", "allreduce=InsAllReduceParallelMesh1DMesh1D;allgather=InsAllGatherParallelMesh1DMesh1D;"
                                              "reducescatter=InsReduceScatterParallelMesh1DMesh1D")
    lib().HcclResetEnvConfigForTest()
    counts = (3, 5000, 300_001)
    rng = np.random.default_rng(5)
    ar_in = {c: [rng.integers(-8, 9, size=c).astype(np.float32) for _ in range(n)] for c in counts}
    ag_in = {c: [rng.integers(-8, 9, size=c).astype(np.float32) for _ in range(n)] for c in counts}
    rs_in = {c: [rng.integers(-8, 9, size=c * n).astype(np.float32) for _ in range(n)] for c in counts}

    def body(comm, rank):
        out, algs = {}, {}
        for c in counts:
            a = ar_in[c][rank].copy()
            comm.all_reduce(a)                               # in place
            comm.synchronize()
            used = [comm.last_algorithm()]
            g = np.empty(c * n, np.float32)
            comm.all_gather(ag_in[c][rank], g)
            comm.synchronize()
            used.append(comm.last_algorithm())
            s = np.empty(c, np.float32)
            comm.reduce_scatter(rs_in[c][rank], s)
            comm.synchronize()
            used.append(comm.last_algorithm())
            algs[c] = used
            out[c] = (a, g, s)
        return out, algs

    try:
        res = run_ranks(n, body, buffer_mb=64)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        monkeypatch.delenv("HCCL_ALGO_NAME", raising=False)
        lib().HcclResetEnvConfigForTest()
    for c in counts:
        want_ar = _oracle(ar_in[c])
        want_ag = np.concatenate(ag_in[c])
        want_rs = _oracle(rs_in[c])
        for r, (out, algs) in enumerate(res):
            a, g, s = out[c]
            assert np.array_equal(a.astype(np.float64), want_ar), (c, r)
            assert np.array_equal(g, want_ag), (c, r)
            assert np.array_equal(s.astype(np.float64), want_rs[r * c:(r + 1) * c]), (c, r)
    big, small = res[0][1][300_001], res[0][1][3]
    if forced:
        assert all("Parallel" in a for a in big + small)
    else:
        assert all("Sequence" in a for a in small)          # nothing to balance in twelve bytes
        if bw:
            for name, used, nbytes in zip(("ALLREDUCE", "ALLGATHER", "REDUCE_SCATTER"), big, (300_001 * 4,) * 3):
                shares, steps, seq, par = plan(name, per, bw[0], servers, bw[1], nbytes)
                gain = par < 0.9 * seq and (min(shares) > 0 or max(steps) > 1)
                assert ("Parallel" in used) == gain, (name, used, shares, steps, seq, par)
            assert any("Parallel" in a for a in big), big


def test_batch_invariant_reduce_scatter_on_two_levels(monkeypatch):
    """HCCL_BIRS_ENABLE=1: the bits of an element of a two-level ReduceScatter do not depend on the count, and they are the bits of
    the fixed tree (rank order inside the server, then server order). Values span twelve decades so that the association shows.
    Without the switch the selector may take the parallel executor, whose cut between the two level orders moves with the count."""
    topo, servers, per = "1x2x4@2,1", 2, 4
    n = servers * per
    monkeypatch.setenv("HCCL_SIM_TOPO", topo)
    monkeypatch.setenv("HCCL_BIRS_ENABLE", "1")
    lib().HcclResetEnvConfigForTest()
    rng = np.random.default_rng(11)
    full = 300_000
    xs = [(rng.standard_normal(full * n) * 10.0 ** rng.integers(-6, 6, full * n)).astype(np.float32) for _ in range(n)]

    def run(count):
        def body(comm, rank):
            out = np.empty(count, np.float32)
            # the first `count` elements of every rank's block
            src = np.concatenate([xs[rank][j * full:j * full + count] for j in range(n)])
            comm.reduce_scatter(src, out)
            comm.synchronize()
            return out, comm.last_algorithm()
        return run_ranks(n, body, buffer_mb=64)

    try:
        big, small = run(full), run(1000)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        monkeypatch.delenv("HCCL_BIRS_ENABLE")
        lib().HcclResetEnvConfigForTest()
    for r in range(n):
        assert "Sequence" in big[r][1] and "Sequence" in small[r][1]
        assert np.array_equal(big[r][0][:1000].view(np.uint32), small[r][0].view(np.uint32))
        # the fixed tree, in numpy: float32 sums inside each server in rank order, then over the servers in order
        blk = [x[r * full:(r + 1) * full] for x in xs]
        partial = []
        for s_ in range(servers):
            acc = blk[s_ * per].copy()
            for j in range(1, per):
                acc = acc + blk[s_ * per + j]
            partial.append(acc)
        want = partial[0]
        for s_ in range(1, servers):
            want = want + partial[s_]
        assert np.array_equal(big[r][0].view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("family", ["Parallel", "Sequence"])
@pytest.mark.parametrize("topo", ["1x2x4", "2x2x2"])
def test_messages_larger_than_the_scratch_run_in_chunks(topo, family, monkeypatch):
    """1 MB of scratch per half against 2.4 MB vectors (AllReduce) and 0.6 MB blocks per rank (AllGather / ReduceScatter, 4.8 MB buffers):
    the multi-level executors cut the call into the largest pieces whose plan fits; a piece of the block forms keeps the stride of
    the whole call."""
    pods, servers, per = (int(v) for v in topo.split("x"))
    n = pods * servers * per
    names = {"Parallel": "allreduce=InsAllReduceParallelMesh1DMesh1D;allgather=InsAllGatherParallelMesh1DMesh1D;reducescatter=InsReduceScatterParallelMesh1DMesh1D",
             "Sequence": "allreduce=InsAllReduceSequenceMesh1DNhr;allgather=InsAllGatherSequenceNhrMesh1D;reducescatter=InsReduceScatterSequenceMesh1DNhr"}[family]
    monkeypatch.setenv("HCCL_SIM_TOPO", topo)
    monkeypatch.setenv("HCCL_ALGO_NAME", names)
    lib().HcclResetEnvConfigForTest()
    rng = np.random.default_rng(41)
    c_ar, c_blk = 600_001, 150_001
    ar_in = [rng.integers(-8, 9, size=c_ar).astype(np.float32) for _ in range(n)]
    ag_in = [rng.integers(-8, 9, size=c_blk).astype(np.float32) for _ in range(n)]
    rs_in = [rng.integers(-8, 9, size=c_blk * n).astype(np.float32) for _ in range(n)]

    def body(comm, rank):
        a = ar_in[rank].copy()
        comm.all_reduce(a)
        comm.synchronize()
        used = [comm.last_algorithm()]
        g = np.empty(c_blk * n, np.float32)
        comm.all_gather(ag_in[rank], g)
        comm.synchronize()
        used.append(comm.last_algorithm())
        s = np.empty(c_blk, np.float32)
        comm.reduce_scatter(rs_in[rank], s)
        comm.synchronize()
        used.append(comm.last_algorithm())
        return a, g, s, used

    try:
        res = run_ranks(n, body, buffer_mb=2)
    finally:
        monkeypatch.delenv("HCCL_SIM_TOPO")
        monkeypatch.delenv("HCCL_ALGO_NAME")
        lib().HcclResetEnvConfigForTest()
    want_ar, want_ag, want_rs = _oracle(ar_in), np.concatenate(ag_in), _oracle(rs_in)
    for r, (a, g, s, used) in enumerate(res):
        assert all(family in u for u in used), used
        assert np.array_equal(a.astype(np.float64), want_ar), r
        assert np.array_equal(g, want_ag), r
        assert np.array_equal(s.astype(np.float64), want_rs[r * c_blk:(r + 1) * c_blk]), r



@pytest.mark.parametrize("topo", [(1, 2, 4), (1, 3, 2), (2, 2, 2)])
def test_chunked_multi_level_plans_pass_the_schedule_checker(topo):
    """160 KB of scratch per half (256 KB with super-pods, whose three-level AllReduce needs 128 KB before the first byte): the checker gets the same pieces the executors run (the largest whose plan fits, found by halving) and
    verifies them together against the whole call, so the block stride of the AllGather / ReduceScatter pieces is checked symbolically."""
    for op, count in (("ALLREDUCE", 100_001), ("ALLGATHER", 17_001), ("REDUCE_SCATTER", 17_001)):
        for family in ("Sequence", "Parallel"):
            alg = {"ALLREDUCE": {"Sequence": "InsAllReduceSequenceMesh1DNhr", "Parallel": "InsAllReduceParallelMesh1DMesh1D"},
                   "ALLGATHER": {"Sequence": "InsAllGatherSequenceNhrMesh1D", "Parallel": "InsAllGatherParallelMesh1DMesh1D"},
                   "REDUCE_SCATTER": {"Sequence": "InsReduceScatterSequenceMesh1DNhr", "Parallel": "InsReduceScatterParallelMesh1DMesh1D"}}[op][family]
            rc, msg = check(op, alg, topo, count, ccl=(256 if topo[0] > 1 else 160) << 10)
            assert rc == 0, (op, alg, msg)
