"""Offline schedule checker over every host-issued algorithm: deadlock freedom, bounds, memory conflicts, semantics --
on flat and simulated multi-server topologies, with boundary sizes (tails, odd rank counts, tiny scratch forcing chunk loops)."""
import ctypes

import pytest

from hccl_b200._lib import lib

CMD = dict(BROADCAST=1, ALLREDUCE=2, REDUCE=3, ALLGATHER=6, REDUCE_SCATTER=7, ALLTOALLV=8, ALLTOALLVC=9, ALLTOALL=10, SCATTER=12,
           BARRIER=14, ALLGATHER_V=15, REDUCE_SCATTER_V=16)
FP32 = 4


def check(op, alg, topo, count, root=0, counts=None, ccl=0):
    l = lib()
    l.HcclCheckAlgorithm.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int,
                                     ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
    l.HcclCheckAlgorithm.restype = ctypes.c_int
    msg = ctypes.create_string_buffer(2048)
    cm = (ctypes.c_uint64 * len(counts))(*counts) if counts else None
    rc = l.HcclCheckAlgorithm(op, alg.encode() if alg else None, topo[0], topo[1], topo[2], count, FP32, root, cm, ccl, msg, 2048)
    return rc, msg.value.decode()


ALGOS = {
    "ALLREDUCE": ["InsAllReduceMesh1DOneShot", "InsAllReduceMesh1DTwoShot", "InsAllReduceRing", "InsAllReduceNHR"],
    "ALLGATHER": ["InsAllGatherMesh1D", "InsAllGatherRing", "InsAllGatherNHR"],
    "REDUCE_SCATTER": ["InsReduceScatterMesh1D", "InsReduceScatterRing", "InsReduceScatterNHR"],
    "BROADCAST": ["InsBroadcastMesh1DOneShot", "InsBroadcastMesh1DTwoShot", "InsBroadcastNHR"],
    "REDUCE": ["ReduceMesh1D", "ReduceMesh1DTwoShot", "ReduceNHR"],
    "SCATTER": ["InsScatterMesh1D", "InsScatterNHR"],
    "ALLTOALL": ["InsAlltoAllMesh1D"],
    "BARRIER": ["InsBarrierMesh1D", "InsBarrierNHR"],
}


@pytest.mark.parametrize("nranks", [2, 3, 4, 5, 7, 8, 16])
@pytest.mark.parametrize("op", list(ALGOS))
def test_flat_algorithms(op, nranks):
    for alg in ALGOS[op]:
        for count in (1, nranks - 1, nranks, 37, 257):
            rc, msg = check(CMD[op], alg, (1, 1, nranks), count, root=nranks - 1)
            assert rc == 0, msg


@pytest.mark.parametrize("nranks", [2, 4, 6])
def test_chunk_loops_with_tiny_scratch(nranks):
    for op in ("ALLREDUCE", "ALLGATHER", "REDUCE_SCATTER", "BROADCAST", "ALLTOALL", "SCATTER", "REDUCE"):
        for alg in ALGOS[op]:
            rc, msg = check(CMD[op], alg, (1, 1, nranks), 5000, root=1, ccl=64 << 10)
            assert rc == 0, msg


@pytest.mark.parametrize("nranks", [2, 3, 5, 8])
def test_variable_count_algorithms(nranks):
    M = [((3 * i + 5 * j) % 4) * 11 + (1 if (i + j) % 3 == 0 else 0) for i in range(nranks) for j in range(nranks)]
    rc, msg = check(CMD["ALLTOALLV"], "InsAlltoAllVMesh1D", (1, 1, nranks), 0, counts=M)
    assert rc == 0, msg
    rc, msg = check(CMD["ALLTOALLVC"], "InsAlltoAllVCMesh1D", (1, 1, nranks), 0, counts=M, ccl=4096 * nranks)   # several credit rounds
    assert rc == 0, msg
    cnts = [(7 * r) % 5 * 13 for r in range(nranks)]
    rc, msg = check(CMD["ALLGATHER_V"], "InsAllGatherVMesh1D", (1, 1, nranks), 0, counts=cnts)
    assert rc == 0, msg
    rc, msg = check(CMD["REDUCE_SCATTER_V"], "InsReduceScatterVMesh1D", (1, 1, nranks), 0, counts=cnts)
    assert rc == 0, msg


@pytest.mark.parametrize("topo", [(1, 2, 2), (1, 2, 4), (1, 3, 2), (1, 4, 2), (2, 2, 2)])
def test_multi_level_sequence_executors(topo):
    n = topo[0] * topo[1] * topo[2]
    for op in ("ALLREDUCE", "ALLGATHER", "REDUCE_SCATTER", "BROADCAST", "REDUCE", "SCATTER", "BARRIER"):
        # with super-pods AllReduce walks three levels; the others fold the upper two into one
        for count in (1, n, 101):
            rc, msg = check(CMD[op], None, topo, count)
            assert rc == 0, msg
            assert "Sequence" in msg


@pytest.mark.parametrize("nranks", [24, 32])
def test_flat_algorithms_at_the_rank_limit(nranks):
    for op, algs in ALGOS.items():
        for alg in algs:
            rc, msg = check(CMD[op], alg, (1, 1, nranks), 1000, root=nranks - 1)
            assert rc == 0, msg


@pytest.mark.parametrize("topo", [(2, 2, 4), (1, 4, 8), (2, 4, 4)])
def test_large_multi_level_allreduce(topo):
    rc, msg = check(CMD["ALLREDUCE"], None, topo, 999)
    assert rc == 0, msg


def test_checker_catches_a_broken_schedule():
    # a scratch window too small for the one-shot slots must be reported as an overrun, not silently accepted
    rc, msg = check(CMD["ALLREDUCE"], "InsAllReduceMesh1DOneShot", (1, 1, 4), 128, ccl=700)
    assert rc != 0


# ---- point-to-point schedules (mailbox slots of `ccl` bytes; a small value forces several rounds through the two slots)
P2P = dict(SEND=4, RECEIVE=5, BATCH_SEND_RECV=13)


@pytest.mark.parametrize("nranks", [2, 3, 5, 8])
@pytest.mark.parametrize("count,slot", [(1, 4096), (1000, 4096), (5000, 4096), (4097, 1024), (64, 256)])
def test_send_receive_schedules(nranks, count, slot):
    for root in (0, nranks - 1):
        rc, msg = check(P2P["SEND"], None, (1, 1, nranks), count, root=root, ccl=slot)
        assert rc == 0, msg


@pytest.mark.parametrize("nranks", [2, 3, 4, 7])
@pytest.mark.parametrize("count,slot", [(2, 4096), (1001, 4096), (6000, 2048), (300, 128)])
def test_batch_send_recv_ring_schedule(nranks, count, slot):
    rc, msg = check(P2P["BATCH_SEND_RECV"], None, (1, 1, nranks), count, ccl=slot)
    assert rc == 0, msg


def test_user_buffer_overrun_is_reported():
    """Bounds are checked for the caller's buffers and the mailbox too, not only for the scratch window: a schedule that
    receives more than the output holds is rejected. The all-gather-v template with counts that disagree with the output
    size the operator defines is such a schedule."""
    l = lib()
    l.HcclCheckPlanText.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32]
    l.HcclCheckPlanText.restype = ctypes.c_int
    msg = ctypes.create_string_buffer(2048)
    # op=AllGather count=4 elems (fp32), 2 ranks; rank 1's write into rank 0's scratch is fine, its final copy overruns OUTPUT
    good = b"op=6 n=2 es=4 count=4 ccl=1024\nr0: COPY out@0 in@0 16; WRITE 1 ccl@0 in@0 16; POST 1 1; WAIT 1 1; COPY out@16 ccl@0 16\n" \
           b"r1: COPY out@16 in@0 16; WRITE 0 ccl@0 in@0 16; POST 0 1; WAIT 0 1; COPY out@0 ccl@0 16\n"
    assert l.HcclCheckPlanText(good, msg, 2048) == 0, msg.value
    bad = good.replace(b"COPY out@16 ccl@0 16", b"COPY out@20 ccl@0 16")
    assert l.HcclCheckPlanText(bad, msg, 2048) != 0 and b"user buffer overrun" in msg.value
    race = good.replace(b"POST 1 1; WAIT 1 1; ", b"").replace(b"POST 0 1; WAIT 0 1; ", b"")
    assert l.HcclCheckPlanText(race, msg, 2048) != 0 and b"memory conflict" in msg.value
    hang = good.replace(b"POST 0 1; ", b"")
    assert l.HcclCheckPlanText(hang, msg, 2048) != 0 and b"deadlock" in msg.value


# ---- the kernels of the SM / NVLS engines, through schedule models built from the real launch lists
SM_ALGOS = {
    "ALLREDUCE": ["SmAllReduceMesh1DOneShot", "SmAllReduceMesh1DTwoShot", "SmAllReduceRing", "NvlsAllReduceOneShot", "NvlsAllReduceTwoShot",
                  "SmAllReduceConcurrent", "NvlsAllReduceConcurrent", "SmAllReduceZeroCopy", "NvlsAllReduceZeroCopy"],
    "ALLGATHER": ["SmAllGatherMesh1D", "SmAllGatherZeroCopy", "NvlsAllGatherZeroCopy"],
    "REDUCE_SCATTER": ["SmReduceScatterMesh1D", "NvlsReduceScatter", "SmReduceScatterZeroCopy", "NvlsReduceScatterZeroCopy"],
    "BROADCAST": ["SmBroadcastMesh1D", "NvlsBroadcast", "SmBroadcastZeroCopy", "NvlsBroadcastZeroCopy"],
    "REDUCE": ["SmReduceMesh1D"],
    "SCATTER": ["SmScatterMesh1D"],
    "ALLTOALL": ["SmAlltoAllMesh1D"],
    "BARRIER": ["SmBarrierMesh1D"],
}


@pytest.mark.parametrize("nranks", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("op", list(SM_ALGOS))
def test_sm_and_nvls_kernel_models(op, nranks):
    for alg in SM_ALGOS[op]:
        for count in (4, 36, 260, 5000):            # multiples of 4 elements: the NVLS kernels take 16-byte multiples
            rc, msg = check(CMD[op], alg, (1, 1, nranks), count, root=nranks - 1, ccl=(1 << 20))
            assert rc == 0, msg


@pytest.mark.parametrize("nranks", [2, 4, 7])
def test_sm_kernel_models_with_chunk_loops(nranks):
    for op in ("ALLREDUCE", "ALLGATHER", "REDUCE_SCATTER", "BROADCAST", "REDUCE", "SCATTER"):
        for alg in SM_ALGOS[op]:
            rc, msg = check(CMD[op], alg, (1, 1, nranks), 9000, root=1, ccl=(192 << 10) if op != "ALLREDUCE" or "Ring" not in alg else (512 << 10))
            assert rc == 0, msg


@pytest.mark.parametrize("nranks", [2, 3, 6])
def test_sm_alltoallv_and_v_forms(nranks):
    import random
    rng = random.Random(nranks)
    cm = [rng.choice([0, 1, 33, 700]) for _ in range(nranks * nranks)]
    for a in range(nranks):
        cm[a * nranks + (a + 1) % nranks] = 0        # a zero row entry per sender
    rc, msg = check(CMD["ALLTOALLV"], "SmAlltoAllVMesh1D", (1, 1, nranks), 0, counts=cm, ccl=(1 << 20))
    assert rc == 0, msg
    # a scratch window of 8 KB: 4 KB are reserved, the rest gives slots of at most 4 KB per pair, so pairs of up to 9000 fp32
    # elements move in up to nine rounds; a zero row, a zero column, and the fixed-size form through the same kernel
    big = [rng.choice([0, 7, 1500, 9000]) for _ in range(nranks * nranks)]
    for j in range(nranks):
        big[(1 % nranks) * nranks + j] = 0
        big[j * nranks + (nranks - 1)] = 0
    rc, msg = check(CMD["ALLTOALLV"], "SmAlltoAllVMesh1D", (1, 1, nranks), 0, counts=big, ccl=(8 << 10))
    assert rc == 0, msg
    rc, msg = check(CMD["ALLTOALL"], "SmAlltoAllMesh1D", (1, 1, nranks), 5000, ccl=(8 << 10))
    assert rc == 0, msg
    rc, msg = check(CMD["ALLTOALLV"], "SmAlltoAllVMesh1D", (1, 1, nranks), 0, counts=big, ccl=(4 << 10))
    assert rc != 0                                     # no room for a slot: refused, not mis-scheduled
    counts = [rng.choice([0, 5, 129, 1000]) for _ in range(nranks)]
    rc, msg = check(CMD["ALLGATHER_V"], "SmAllGatherVMesh1D", (1, 1, nranks), 0, counts=counts, ccl=(1 << 20))
    assert rc == 0, msg
    rc, msg = check(CMD["REDUCE_SCATTER_V"], "SmReduceScatterVMesh1D", (1, 1, nranks), 0, counts=counts, ccl=(1 << 20))
    assert rc == 0, msg


PIPELINED = {
    "ALLREDUCE": ["SmAllReducePipelined", "NvlsAllReducePipelined"],
    "REDUCE_SCATTER": ["SmReduceScatterPipelined", "NvlsReduceScatterPipelined"],
    "ALLGATHER": ["SmAllGatherPush", "NvlsAllGatherPush"],
    "BROADCAST": ["SmBroadcastPush", "NvlsBroadcastPush"],
    "ALLTOALL": ["SmAlltoAllPush"],
}


@pytest.mark.parametrize("nranks", [2, 4, 5])
def test_pipelined_kernel_models(nranks):
    """The warp-specialised pipelines as three queues per channel: deadlock freedom of the STAGED / MOVED / DRAINED protocol, ring slots
    inside the scratch window, no slot rewritten while a peer may still read it, and the operator's result -- over one sub-chunk, a few,
    and many trips round the two-deep ring."""
    for op, algs in PIPELINED.items():
        for alg in algs:
            for count, ccl in ((5, 256 << 10), (4099, 256 << 10), (60_001, 64 << 10)):
                if alg.startswith("Nvls") and (count * 4) % 16:
                    count += 4 - count % 4                     # the switch forms take whole 16-byte vectors
                rc, msg = check(CMD[op], alg, (1, 1, nranks), count, root=nranks - 1, ccl=ccl)
                assert rc == 0, (alg, count, msg)


def test_pipelined_model_walks_the_longest_part_of_any_slice():
    """Counts at which the last channel's part of the (shorter) last slice needs one sub-chunk more than its part of the first slice:
    a loop sized by the first slice alone would leave the tail of the buffer unreduced, and the checker would report a wrong result."""
    rc, msg = check(CMD["ALLREDUCE"], "SmAllReducePipelined", (1, 1, 4), 311_873, ccl=256 << 10)
    assert rc == 0, msg
    rc, msg = check(CMD["ALLREDUCE"], "SmAllReducePipelined", (1, 1, 3), 101_121, ccl=64 << 10)
    assert rc == 0, msg


def test_random_geometries_of_every_kernel_model():
    """Random rank counts, element counts and scratch sizes for every SM / NVLS / pipelined algorithm: the model of each kernel restates
    its index arithmetic, so an off-by-one in slices, parts, sub-chunks or chunk loops shows up as a wrong element, an overrun or a race.
    A scratch window that is too small for an algorithm must be refused by the planner (a non-zero status without a verdict on the
    schedule), never mis-scheduled."""
    from hypothesis import given, settings, strategies as st

    every = [(op, a) for op, algs in SM_ALGOS.items() for a in algs] + [(op, a) for op, algs in PIPELINED.items() for a in algs]

    @settings(max_examples=120, deadline=None)
    @given(st.sampled_from(every), st.integers(2, 8), st.integers(1, 30_000), st.sampled_from([32 << 10, 96 << 10, 256 << 10, 1 << 20]), st.integers(0, 7))
    def prop(case, nranks, count, ccl, root):
        op, alg = case
        if alg.startswith("Nvls") or "ZeroCopy" in alg:
            count = (count + 3) // 4 * 4                      # whole 16-byte vectors of fp32
        rc, msg = check(CMD[op], alg, (1, 1, nranks), count, root=root % nranks, ccl=ccl)
        if rc != 0:
            # refusals are fine (window too small, shape not supported); verdicts about the schedule are not
            assert not any(w in msg for w in ("semantic error", "conflict", "overrun", "deadlock", "never waited", "disagree")), (alg, nranks, count, ccl, msg)

    prop()


def test_random_count_matrices_of_the_variable_forms():
    """AlltoAllV with random count matrices (zeros included) through scratch windows small enough for several rounds, and the V forms of
    AllGather / ReduceScatter on the mesh and the pipelined kernels with random per-rank counts."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=80, deadline=None)
    @given(st.integers(2, 8), st.data())
    def prop(nranks, data):
        cell = st.sampled_from([0, 0, 1, 3, 100, 1029, 7000])
        cm = data.draw(st.lists(cell, min_size=nranks * nranks, max_size=nranks * nranks))
        ccl = data.draw(st.sampled_from([8 << 10, 24 << 10, 1 << 20]))
        rc, msg = check(CMD["ALLTOALLV"], "SmAlltoAllVMesh1D", (1, 1, nranks), 0, counts=cm, ccl=ccl)
        assert rc == 0 or not any(w in msg for w in ("semantic error", "conflict", "overrun", "deadlock", "never waited", "disagree")), (nranks, cm, ccl, msg)
        counts = data.draw(st.lists(cell, min_size=nranks, max_size=nranks))
        for op, alg in (("ALLGATHER_V", "SmAllGatherVMesh1D"), ("REDUCE_SCATTER_V", "SmReduceScatterVMesh1D"), ("ALLGATHER_V", "SmAllGatherVPush"),
                        ("REDUCE_SCATTER_V", "SmReduceScatterVPipelined")):
            rc, msg = check(CMD[op], alg, (1, 1, nranks), 0, counts=counts, ccl=256 << 10)
            assert rc == 0 or not any(w in msg for w in ("semantic error", "conflict", "overrun", "deadlock", "never waited", "disagree")), (alg, nranks, counts, msg)

    prop()
