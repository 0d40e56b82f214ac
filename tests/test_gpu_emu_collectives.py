"""SM-engine collective kernels on ONE GPU: all ranks emulated in a single cooperative launch (blockIdx.y = rank).
Numerics are compared with a plain PyTorch fp32/fp64 reference of the same operator."""
import pytest
import torch

from hccl_b200.types import ReduceOp

pytestmark = pytest.mark.gpu

CMD = dict(BROADCAST=1, ALLREDUCE=2, REDUCE=3, ALLGATHER=6, REDUCE_SCATTER=7, ALLTOALLV=8, ALLTOALLVC=9, ALLTOALL=10, SCATTER=12,
           BARRIER=14, ALLGATHER_V=15, REDUCE_SCATTER_V=16)


@pytest.fixture(scope="module")
def emu_mod():
    from hccl_b200.utils import emu
    return emu


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(dtype)
    return torch.randint(-50, 50, (n,), generator=g, device="cuda", dtype=torch.int64).to(dtype)


def _ref_reduce(xs, op, dtype):
    acc = torch.stack([x.to(torch.float64) if dtype.is_floating_point else x.to(torch.int64) for x in xs])
    if op == ReduceOp.SUM:
        r = acc.sum(0)
    elif op == ReduceOp.PROD:
        r = acc.prod(0)
    elif op == ReduceOp.MAX:
        r = acc.max(0).values
    else:
        r = acc.min(0).values
    return r


def _tol(dtype, n):
    if dtype == torch.bfloat16:
        return 2e-2 * n ** 0.5
    if dtype == torch.float16:
        return 3e-3 * n ** 0.5
    if dtype == torch.float32:
        return 1e-5 * n
    return 0


@pytest.mark.parametrize("nranks", [2, 3, 4, 8])
@pytest.mark.parametrize("alg", ["SmAllReduceMesh1DOneShot", "SmAllReduceMesh1DTwoShot"])
@pytest.mark.parametrize("count", [1, 7, 1024, 4099, 65536 + 3])
def test_allreduce_fp32_sum(emu_mod, nranks, alg, count):
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        xs = [_rand(count, torch.float32, 100 + r) for r in range(nranks)]
        outs = [torch.empty_like(x) for x in xs]
        assert w.run(CMD["ALLREDUCE"], alg, xs, outs, count, torch.float32) == 0
        ref = _ref_reduce(xs, ReduceOp.SUM, torch.float32)
        for o in outs:
            assert torch.allclose(o.double(), ref, atol=_tol(torch.float32, nranks), rtol=1e-5)
            assert torch.equal(o, outs[0])   # rank-order reduction: identical bits on every rank


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.int8, torch.float64, torch.int16])
@pytest.mark.parametrize("op", [ReduceOp.SUM, ReduceOp.MAX, ReduceOp.MIN])
def test_allreduce_dtypes_ops(emu_mod, dtype, op):
    nranks, count = 4, 3001
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        for alg in ("SmAllReduceMesh1DOneShot", "SmAllReduceMesh1DTwoShot"):
            xs = [_rand(count, dtype, 7 + r) for r in range(nranks)]
            outs = [torch.empty_like(x) for x in xs]
            assert w.run(CMD["ALLREDUCE"], alg, xs, outs, count, dtype, op) == 0
            ref = _ref_reduce(xs, op, dtype)
            for o in outs:
                if dtype.is_floating_point:
                    assert torch.allclose(o.double(), ref, atol=_tol(dtype, nranks), rtol=1e-2 if dtype != torch.float64 else 1e-12)
                else:
                    assert torch.equal(o.to(torch.int64), ref.to(dtype).to(torch.int64))


@pytest.mark.parametrize("dtype", [torch.uint8, torch.uint16, torch.uint32])
def test_allreduce_unsigned(emu_mod, dtype):
    nranks, count = 4, 2051
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        xs64 = [torch.randint(0, 60, (count,), device="cuda", dtype=torch.int64) for _ in range(nranks)]
        xs = [x.to(dtype) for x in xs64]
        for op, ref in ((ReduceOp.SUM, torch.stack(xs64).sum(0)), (ReduceOp.MAX, torch.stack(xs64).max(0).values)):
            outs = [torch.empty_like(x) for x in xs]
            assert w.run(CMD["ALLREDUCE"], "SmAllReduceMesh1DTwoShot", xs, outs, count, dtype, op) == 0
            for o in outs:
                assert torch.equal(o.to(torch.int64), ref)


def test_allreduce_prod_and_inplace(emu_mod):
    nranks, count = 3, 513
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        xs = [(_rand(count, torch.float32, r) * 0.5 + 1.0) for r in range(nranks)]
        ref = _ref_reduce(xs, ReduceOp.PROD, torch.float32)
        bufs = [x.clone() for x in xs]
        assert w.run(CMD["ALLREDUCE"], "SmAllReduceMesh1DTwoShot", bufs, bufs, count, torch.float32, ReduceOp.PROD) == 0
        for b in bufs:
            assert torch.allclose(b.double(), ref, rtol=1e-5)


def test_allreduce_chunk_loop_and_back_to_back(emu_mod):
    """Scratch smaller than the payload forces several launches; repeated calls exercise the ping-pong halves."""
    nranks, count = 4, 300_000
    with emu_mod.EmuWorld(nranks, 256 << 10) as w:
        for it in range(3):
            xs = [_rand(count, torch.float32, 50 * it + r) for r in range(nranks)]
            outs = [torch.empty_like(x) for x in xs]
            alg = "SmAllReduceMesh1DTwoShot" if it != 1 else "SmAllReduceMesh1DOneShot"
            assert w.run(CMD["ALLREDUCE"], alg, xs, outs, count, torch.float32) == 0
            ref = _ref_reduce(xs, ReduceOp.SUM, torch.float32)
            for o in outs:
                assert torch.allclose(o.double(), ref, atol=1e-4)


@pytest.mark.parametrize("nranks", [2, 5, 8])
def test_allgather_reducescatter(emu_mod, nranks):
    count = 2049
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        xs = [_rand(count, torch.bfloat16, r) for r in range(nranks)]
        outs = [torch.empty(count * nranks, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLGATHER"], "SmAllGatherMesh1D", xs, outs, count, torch.bfloat16) == 0
        want = torch.cat(xs)
        for o in outs:
            assert torch.equal(o, want)
        full = [_rand(count * nranks, torch.float32, 10 + r) for r in range(nranks)]
        rs = [torch.empty(count, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["REDUCE_SCATTER"], "SmReduceScatterMesh1D", full, rs, count, torch.float32) == 0
        ref = _ref_reduce(full, ReduceOp.SUM, torch.float32)
        for r in range(nranks):
            assert torch.allclose(rs[r].double(), ref[r * count:(r + 1) * count], atol=1e-4)


@pytest.mark.parametrize("root", [0, 2])
def test_broadcast_reduce_scatter_rooted(emu_mod, root):
    nranks, count = 4, 5000
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        bufs = [_rand(count, torch.float32, r) for r in range(nranks)]
        want = bufs[root].clone()
        assert w.run(CMD["BROADCAST"], "SmBroadcastMesh1D", bufs, bufs, count, torch.float32, root=root) == 0
        for b in bufs:
            assert torch.equal(b, want)
        xs = [_rand(count, torch.float32, 20 + r) for r in range(nranks)]
        outs = [torch.zeros(count, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["REDUCE"], "SmReduceMesh1D", xs, outs, count, torch.float32, root=root) == 0
        assert torch.allclose(outs[root].double(), _ref_reduce(xs, ReduceOp.SUM, torch.float32), atol=1e-4)
        send = [_rand(count * nranks, torch.float32, 30 + r) for r in range(nranks)]
        recv = [torch.zeros(count, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["SCATTER"], "SmScatterMesh1D", send, recv, count, torch.float32, root=root) == 0
        for r in range(nranks):
            assert torch.equal(recv[r], send[root][r * count:(r + 1) * count])


@pytest.mark.parametrize("nranks", [3, 4, 8])
def test_alltoall_and_v(emu_mod, nranks):
    count = 777
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        send = [_rand(count * nranks, torch.float32, r) for r in range(nranks)]
        recv = [torch.zeros(count * nranks, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLTOALL"], "SmAlltoAllMesh1D", send, recv, count, torch.float32) == 0
        for r in range(nranks):
            for s in range(nranks):
                assert torch.equal(recv[r][s * count:(s + 1) * count], send[s][r * count:(r + 1) * count])
        # variable counts, including zeros
        M = [[(3 * i + 5 * j) % 7 * 100 + (0 if (i + j) % 3 else 1) * 13 for j in range(nranks)] for i in range(nranks)]
        M[1][2] = 0
        sends = [_rand(max(1, sum(M[i])), torch.float32, 40 + i) for i in range(nranks)]
        recvs = [torch.zeros(max(1, sum(M[j][i] for j in range(nranks))), dtype=torch.float32, device="cuda") for i in range(nranks)]
        flat = [v for row in M for v in row]
        assert w.run(CMD["ALLTOALLV"], "SmAlltoAllVMesh1D", sends, recvs, 0, torch.float32, counts=flat) == 0
        for i in range(nranks):
            ro = 0
            for j in range(nranks):
                so = sum(M[j][:i])
                assert torch.equal(recvs[i][ro:ro + M[j][i]], sends[j][so:so + M[j][i]])
                ro += M[j][i]


@pytest.mark.parametrize("nranks", [4, 8])
def test_alltoallv_zero_row_zero_column_and_pairs_above_the_scratch_half(emu_mod, nranks):
    """One rank sends nothing, one rank receives nothing, and some pairs carry more than half of the scratch window
    (64 KB window here, pairs of up to 100 KB), so the kernel has to loop over credit rounds with uneven pair lengths."""
    M = [[(5000 * ((i + 2 * j) % 4) + 17 * (i + 1)) for j in range(nranks)] for i in range(nranks)]
    M[0][3] = 25_000                                   # 100 KB of fp32 in one pair
    M[3][0] = 1
    for j in range(nranks):
        M[1][j] = 0                                    # rank 1 sends nothing
        M[j][2] = 0                                    # rank 2 receives nothing
    with emu_mod.EmuWorld(nranks, 64 << 10) as w:
        sends = [_rand(max(1, sum(M[i])), torch.float32, 140 + i) for i in range(nranks)]
        recvs = [torch.full((max(1, sum(M[j][i] for j in range(nranks))),), -7.0, dtype=torch.float32, device="cuda") for i in range(nranks)]
        flat = [v for row in M for v in row]
        assert w.run(CMD["ALLTOALLV"], "SmAlltoAllVMesh1D", sends, recvs, 0, torch.float32, counts=flat) == 0
        for i in range(nranks):
            ro = 0
            for j in range(nranks):
                so = sum(M[j][:i])
                assert torch.equal(recvs[i][ro:ro + M[j][i]], sends[j][so:so + M[j][i]]), (i, j)
                ro += M[j][i]
        assert torch.all(recvs[2] == -7.0)             # nothing was written to the rank that receives nothing


def test_allgatherv_reducescatterv(emu_mod):
    nranks = 4
    counts = [100, 0, 1025, 33]
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        xs = [_rand(max(1, counts[r]), torch.float32, r) for r in range(nranks)]
        outs = [torch.zeros(sum(counts), dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLGATHER_V"], "SmAllGatherVMesh1D", xs, outs, 0, torch.float32, counts=counts) == 0
        want = torch.cat([xs[r][:counts[r]] for r in range(nranks)])
        for o in outs:
            assert torch.equal(o, want)
        full = [_rand(sum(counts), torch.float32, 60 + r) for r in range(nranks)]
        rs = [torch.zeros(max(1, counts[r]), dtype=torch.float32, device="cuda") for r in range(nranks)]
        assert w.run(CMD["REDUCE_SCATTER_V"], "SmReduceScatterVMesh1D", full, rs, 0, torch.float32, counts=counts) == 0
        ref = _ref_reduce(full, ReduceOp.SUM, torch.float32)
        off = 0
        for r in range(nranks):
            assert torch.allclose(rs[r][:counts[r]].double(), ref[off:off + counts[r]], atol=1e-4)
            off += counts[r]


def test_batch_send_recv_ring_and_barrier(emu_mod):
    nranks = 4
    with emu_mod.EmuWorld(nranks, 1 << 20) as w:
        n = 200_000   # several mailbox rounds
        src = [_rand(n, torch.float32, r) for r in range(nranks)]
        dst = [torch.zeros(n, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        transfers = [(r, (r + 1) % nranks, src[r], dst[(r + 1) % nranks]) for r in range(nranks)]
        assert w.batch_send_recv(transfers) == 0
        for r in range(nranks):
            assert torch.equal(dst[(r + 1) % nranks], src[r])
        # a second round reuses the mailbox sequence numbers
        dst2 = [torch.zeros(1000, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.batch_send_recv([(0, 3, src[0][:1000], dst2[3]), (3, 0, src[3][:1000], dst2[0])]) == 0
        assert torch.equal(dst2[3], src[0][:1000]) and torch.equal(dst2[0], src[3][:1000])
        assert w.run(CMD["BARRIER"], "SmBarrierMesh1D", None, None, 0, torch.int8) == 0


def test_bounded_wait_reports_timeout(emu_mod):
    """A rank whose peers never arrive gives up after the deadline, records who it waited for, and the context stays
    usable (the next operator on a cleared world succeeds)."""
    with emu_mod.EmuWorld(2, 1 << 20, wait_timeout_ms=200) as w:
        assert w.lonely_barrier(0) == 9   # HCCL_E_TIMEOUT
        st = w.status(0, clear=True)
        assert st[0] == 1 and st[1] == 0 and st[2] == 1   # code, rank, peer
        xs = [_rand(100, torch.float32, r) for r in range(2)]
        outs = [torch.empty_like(x) for x in xs]
        assert w.run(CMD["ALLREDUCE"], "SmAllReduceMesh1DOneShot", xs, outs, 100, torch.float32) == 0
        assert torch.allclose(outs[0], xs[0] + xs[1])


# ---- warp-specialised pipelined kernels (plain peer-memory variants; the NVLS variants need a real multicast mapping) ----
@pytest.mark.parametrize("nranks,ccl_kb,ctas,count", [(n, c, g, k) for (n, c, g) in [(2, 1024, 4), (4, 256, 4), (8, 256, 2), (3, 64, 3)] for k in [1, 37, 4099, 300_001]] +
                         # 12 MB through 4 KB sub-chunks: 193 trips round the ring per channel; and the grid / scratch a 4-rank job with a 4 MB buffer gets
                         [(4, 256, 4, (3 << 20) + 5), (4, 4096, 32, (3 << 20) + 5), (4, 2048, 32, (3 << 20) + 5),
                          # counts where the last channel's part of the (shorter) last slice needs one sub-chunk more than its part of slice 0
                          (4, 256, 4, 311_873), (3, 64, 3, 101_121)])
def test_pipelined_allreduce(emu_mod, nranks, ccl_kb, ctas, count):
    """Small scratch + large count walks the ring many times (sub-chunks of a few KB), which exercises slot reuse."""
    with emu_mod.EmuWorld(nranks, ccl_kb << 10) as w:
        for it, (dtype, op) in enumerate(((torch.float32, ReduceOp.SUM), (torch.bfloat16, ReduceOp.MAX), (torch.int32, ReduceOp.SUM))):
            xs = [_rand(count, dtype, 300 + 10 * it + r) for r in range(nranks)]
            outs = [torch.empty_like(x) for x in xs]
            assert w.run(CMD["ALLREDUCE"], "SmAllReducePipelined", xs, outs, count, dtype, op, max_ctas=ctas) == 0
            ref = _ref_reduce(xs, op, dtype)
            for o in outs:
                if dtype.is_floating_point:
                    assert torch.allclose(o.double(), ref, atol=_tol(dtype, nranks), rtol=1e-2)
                else:
                    assert torch.equal(o.to(torch.int64), ref)
                assert torch.equal(o, outs[0])


@pytest.mark.parametrize("nranks", [2, 5, 8])
@pytest.mark.parametrize("count", [3, 2049, 150_001])
def test_pipelined_allgather_reducescatter(emu_mod, nranks, count):
    with emu_mod.EmuWorld(nranks, 256 << 10) as w:
        for it in range(2):                                   # back-to-back operators: flag bases carry over
            xs = [_rand(count, torch.bfloat16, 7 * it + r) for r in range(nranks)]
            outs = [torch.empty(count * nranks, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
            assert w.run(CMD["ALLGATHER"], "SmAllGatherPush", xs, outs, count, torch.bfloat16, max_ctas=3) == 0
            want = torch.cat(xs)
            for o in outs:
                assert torch.equal(o, want)
            full = [_rand(count * nranks, torch.float32, 10 + r + it) for r in range(nranks)]
            rs = [torch.empty(count, dtype=torch.float32, device="cuda") for _ in range(nranks)]
            assert w.run(CMD["REDUCE_SCATTER"], "SmReduceScatterPipelined", full, rs, count, torch.float32, max_ctas=3) == 0
            ref = _ref_reduce(full, ReduceOp.SUM, torch.float32)
            for r in range(nranks):
                assert torch.allclose(rs[r].double(), ref[r * count:(r + 1) * count], atol=1e-4)


def test_pipelined_v_forms_and_unaligned_input(emu_mod):
    nranks = 4
    counts = [100, 0, 70_001, 33]
    with emu_mod.EmuWorld(nranks, 128 << 10) as w:
        xs = [_rand(max(1, counts[r]) + 1, torch.float32, r)[1:] for r in range(nranks)]       # 4-byte aligned only
        outs = [torch.zeros(sum(counts), dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLGATHER_V"], "SmAllGatherVPush", xs, outs, 0, torch.float32, counts=counts, max_ctas=2) == 0
        want = torch.cat([xs[r][:counts[r]] for r in range(nranks)])
        for o in outs:
            assert torch.equal(o, want)
        full = [_rand(sum(counts), torch.float32, 60 + r) for r in range(nranks)]
        rs = [torch.zeros(max(1, counts[r]), dtype=torch.float32, device="cuda") for r in range(nranks)]
        assert w.run(CMD["REDUCE_SCATTER_V"], "SmReduceScatterVPipelined", full, rs, 0, torch.float32, counts=counts, max_ctas=2) == 0
        ref = _ref_reduce(full, ReduceOp.SUM, torch.float32)
        off = 0
        for r in range(nranks):
            assert torch.allclose(rs[r][:counts[r]].double(), ref[off:off + counts[r]], atol=1e-4)
            off += counts[r]
        # one-byte elements at an odd address
        b = [torch.randint(0, 255, (10_001,), device="cuda", dtype=torch.uint8)[1:] for _ in range(nranks)]
        bo = [torch.zeros(10_000 * nranks, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLGATHER"], "SmAllGatherPush", b, bo, 10_000, torch.uint8, max_ctas=2) == 0
        for o in bo:
            assert torch.equal(o, torch.cat(b))


@pytest.mark.parametrize("nranks", [2, 4, 7])
@pytest.mark.parametrize("count", [5, 4099, 120_001])
def test_pipelined_broadcast_and_alltoall(emu_mod, nranks, count):
    with emu_mod.EmuWorld(nranks, 128 << 10) as w:
        for root in (0, nranks - 1):
            bufs = [_rand(count, torch.float32, 900 + r) for r in range(nranks)]
            want = bufs[root].clone()
            assert w.run(CMD["BROADCAST"], "SmBroadcastPush", bufs, bufs, count, torch.float32, root=root, max_ctas=3) == 0
            for b in bufs:
                assert torch.equal(b, want)
        send = [_rand(count * nranks, torch.float32, 950 + r) for r in range(nranks)]
        recv = [torch.zeros(count * nranks, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLTOALL"], "SmAlltoAllPush", send, recv, count, torch.float32, max_ctas=3) == 0
        for r in range(nranks):
            for s in range(nranks):
                assert torch.equal(recv[r][s * count:(s + 1) * count], send[s][r * count:(r + 1) * count])


@pytest.mark.parametrize("nranks", [2, 3, 4, 8])
@pytest.mark.parametrize("count", [1, 37, 4099, 200_003])
def test_ring_allreduce(emu_mod, nranks, count):
    """Ring reduce-scatter + all-gather on the SM engine (the comparator for the mesh kernels); small scratch forces the chunk loop."""
    with emu_mod.EmuWorld(nranks, 256 << 10) as w:
        for dtype, op in ((torch.float32, ReduceOp.SUM), (torch.bfloat16, ReduceOp.MAX), (torch.int32, ReduceOp.SUM)):
            xs = [_rand(count, dtype, 500 + r) for r in range(nranks)]
            bufs = [x.clone() for x in xs]
            assert w.run(CMD["ALLREDUCE"], "SmAllReduceRing", bufs, bufs, count, dtype, op, max_ctas=3) == 0      # in place
            ref = _ref_reduce(xs, op, dtype)
            for b in bufs:
                if dtype.is_floating_point:
                    assert torch.allclose(b.double(), ref, atol=_tol(dtype, nranks), rtol=1e-2)
                else:
                    assert torch.equal(b.to(torch.int64), ref)
                assert torch.equal(b, bufs[0])


def test_device_trace_records_every_kernel(emu_mod):
    """CTA 0 of every collective kernel stamps a record from the GPU's %globaltimer: entry, its first and last all-rank
    synchronisation, exit. Records follow the device op counter, and a kernel that gave up waiting has no exit stamp."""
    with emu_mod.EmuWorld(4, 1 << 20, wait_timeout_ms=200) as w:
        xs = [_rand(30_000, torch.float32, r) for r in range(4)]      # 120 KB per rank: one launch per operator with 1 MB of scratch
        outs = [torch.empty_like(x) for x in xs]
        for alg, syncs in (("SmAllReduceMesh1DOneShot", 1), ("SmAllReduceMesh1DTwoShot", 2), ("SmAllReduceMesh1DTwoShot", 2)):
            assert w.run(CMD["ALLREDUCE"], alg, xs, outs, 30_000, torch.float32, max_ctas=4) == 0
        for rank in range(4):
            recs = w.trace(rank)
            assert [r["seq"] for r in recs] == [0, 1, 2]
            assert [r["syncs"] for r in recs] == [1, 2, 2]
            for r in recs:
                assert 0 < r["enter"] <= r["first_sync"] <= r["last_sync"] <= r["leave"]
                assert r["leave"] - r["enter"] < 50_000_000          # a 120 KB all-reduce takes microseconds, not 50 ms
            assert recs[0]["leave"] <= recs[1]["enter"] + 1_000_000 and recs[1]["enter"] < recs[2]["enter"]
        assert w.lonely_barrier(1) == 9
        last = w.trace(1)[-1]
        assert last["seq"] == 3 and last["leave"] == 0 and last["syncs"] == 0
        w.status(1, clear=True)


@pytest.mark.parametrize("ratio", [None, "1:1", "3:1", "1:5", "1:0"])
@pytest.mark.parametrize("nranks,count", [(2, 64), (4, 100_003), (8, 1_000_000), (3, 4097)])
def test_concurrent_allreduce_splits_one_payload_between_two_sub_grids(emu_mod, monkeypatch, ratio, nranks, count):
    """Two all-reduce algorithms share one launch: the first CTAs take the first part of the payload, the rest the remainder,
    each in its own scratch region, in the proportion HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO gives. Without a multicast
    mapping (emulated ranks) both parts run the peer-store two-shot, whose result is bit-identical to the plain two-shot."""
    from hccl_b200._lib import lib
    if ratio is None:
        monkeypatch.delenv("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", raising=False)
    else:
        monkeypatch.setenv("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", ratio)
    lib().HcclResetEnvConfigForTest()
    try:
        with emu_mod.EmuWorld(nranks, 1 << 20) as w:        # 1 MB scratch: the 4 MB payload also walks the chunk loop
            for dtype in (torch.float32, torch.bfloat16):
                xs = [_rand(count, dtype, 40 + r) for r in range(nranks)]
                outs = [torch.empty_like(x) for x in xs]
                ref = [torch.empty_like(x) for x in xs]
                assert w.run(CMD["ALLREDUCE"], "SmAllReduceConcurrent", xs, outs, count, dtype, ReduceOp.SUM, max_ctas=6) == 0
                assert w.run(CMD["ALLREDUCE"], "SmAllReduceMesh1DTwoShot", xs, ref, count, dtype, ReduceOp.SUM, max_ctas=6) == 0
                for o, r in zip(outs, ref):
                    assert torch.equal(o, r)
    finally:
        monkeypatch.delenv("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", raising=False)
        lib().HcclResetEnvConfigForTest()


@pytest.mark.parametrize("nranks,count", [(2, 64), (4, 40_000), (8, 262_144), (3, 4100)])
def test_zero_copy_kernels_on_registered_windows(emu_mod, nranks, count):
    """Buffers at the same heap offset on every rank (registered windows): peers read and write them directly, the scratch
    buffer is not used at all -- it is far too small here for the payloads -- and results match the staged kernels' bit for bit."""
    es = 4
    with emu_mod.EmuWorld(nranks, 64 << 10, arena_bytes=(2 * nranks + 4) * count * es + (1 << 20)) as w:
        big_in = [w.arena_tensor(r, 0, count * nranks, torch.float32) for r in range(nranks)]
        big_out = [w.arena_tensor(r, (count * nranks * es + 255) // 256 * 256, count * nranks, torch.float32) for r in range(nranks)]
        # all-reduce, out of place and in place
        for it in range(2):
            xs = [_rand(count, torch.float32, 60 + it * 10 + r) for r in range(nranks)]
            for r in range(nranks):
                big_in[r][:count].copy_(xs[r])
            ins = [t[:count] for t in big_in]
            outs = [t[:count] for t in (big_out if it == 0 else big_in)]
            ref = [torch.empty_like(x) for x in xs]
            with emu_mod.EmuWorld(nranks, 8 << 20) as staged:
                assert staged.run(CMD["ALLREDUCE"], "SmAllReduceMesh1DTwoShot", xs, ref, count, torch.float32, ReduceOp.SUM) == 0
            assert w.run(CMD["ALLREDUCE"], "SmAllReduceZeroCopy", ins, outs, count, torch.float32, ReduceOp.SUM, max_ctas=4) == 0
            for o, rf in zip(outs, ref):
                assert torch.equal(o, rf)
        # reduce-scatter: registered input, plain output
        full = [_rand(count * nranks, torch.float32, 80 + r) for r in range(nranks)]
        for r in range(nranks):
            big_in[r].copy_(full[r])
        outs = [torch.empty(count, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["REDUCE_SCATTER"], "SmReduceScatterZeroCopy", big_in, outs, count, torch.float32, ReduceOp.SUM, max_ctas=4) == 0
        acc = full[0].clone()
        for r in range(1, nranks):
            acc += full[r]
        for r in range(nranks):
            assert torch.equal(outs[r], acc[r * count:(r + 1) * count])      # rank order, fp32: the same sum order as here
        # all-gather: plain input, registered output
        xs = [_rand(count, torch.float32, 90 + r) for r in range(nranks)]
        assert w.run(CMD["ALLGATHER"], "SmAllGatherZeroCopy", xs, big_out, count, torch.float32, max_ctas=4) == 0
        for r in range(nranks):
            assert torch.equal(big_out[r], torch.cat(xs))
        # broadcast in the registered window
        root = nranks - 1
        src = _rand(count, torch.float32, 99)
        for r in range(nranks):
            big_out[r][:count].copy_(src if r == root else torch.zeros_like(src))
        bufs = [t[:count] for t in big_out]
        assert w.run(CMD["BROADCAST"], "SmBroadcastZeroCopy", bufs, bufs, count, torch.float32, root=root, max_ctas=4) == 0
        for r in range(nranks):
            assert torch.equal(bufs[r], src)
        # a buffer outside the arena is refused (HCCL_E_NOT_SUPPORT), not staged silently under this algorithm name
        outside = [torch.zeros(count, device="cuda") for _ in range(nranks)]
        assert w.run(CMD["ALLREDUCE"], "SmAllReduceZeroCopy", outside, outside, count, torch.float32, ReduceOp.SUM) == 5
