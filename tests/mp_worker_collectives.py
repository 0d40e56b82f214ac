"""Worker of the multi-GPU collective tests (one process per GPU, started by torchrun). Every rank can regenerate every
rank's input (seeded by rank), so expected results are computed locally in fp64/int64 without another library."""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
import hccl_b200  # noqa: E402
from hccl_b200.comm import init_from_env  # noqa: E402
from hccl_b200.types import ReduceOp  # noqa: E402


def gen(rank, n, dtype, salt=0):
    g = torch.Generator(device="cuda").manual_seed(1000 * rank + salt)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
    return torch.randint(-40, 40, (n,), generator=g, device="cuda", dtype=torch.int64).to(dtype)


def ref_reduce(world, n, dtype, op, salt=0):
    acc = torch.stack([gen(r, n, dtype, salt).to(torch.float64 if dtype.is_floating_point else torch.int64) for r in range(world)])
    return {ReduceOp.SUM: lambda: acc.sum(0), ReduceOp.MAX: lambda: acc.max(0).values, ReduceOp.MIN: lambda: acc.min(0).values,
            ReduceOp.PROD: lambda: acc.prod(0)}[op]()


def close(out, ref, dtype, world):
    if not dtype.is_floating_point:
        return torch.equal(out.to(torch.int64), ref.to(dtype).to(torch.int64))
    tol = {torch.bfloat16: 3e-2, torch.float16: 4e-3, torch.float32: 1e-5, torch.float64: 1e-12}[dtype] * world
    return torch.allclose(out.double(), ref, atol=tol, rtol=tol)


def main():
    comm = init_from_env()
    rank, world = comm.rank, comm.size
    fails = []

    def check(name, ok):
        if not ok:
            fails.append(name)
            print(f"[rank {rank}] FAIL {name}", flush=True)

    sizes = [1, 33, 1024, 65537, 1 << 20, (3 << 20) + 5]
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64):
        for n in sizes if dtype in (torch.float32, torch.bfloat16) else sizes[:4]:
            for op in (ReduceOp.SUM, ReduceOp.MAX):
                x = gen(rank, n, dtype)
                out = torch.empty_like(x)
                comm.all_reduce(x, out, op)
                torch.cuda.synchronize()
                check(f"allreduce {dtype} n={n} {op.name}", close(out, ref_reduce(world, n, dtype, op), dtype, world))
    # in place + repeated calls (ping-pong halves, plan reuse)
    for it in range(4):
        x = gen(rank, 50_000, torch.float32, salt=it)
        comm.all_reduce(x)
        torch.cuda.synchronize()
        check(f"allreduce inplace it={it}", close(x, ref_reduce(world, 50_000, torch.float32, ReduceOp.SUM, salt=it), torch.float32, world))
    for n in (5, 4096, 300_001):
        x = gen(rank, n, torch.bfloat16)
        out = torch.empty(n * world, dtype=torch.bfloat16, device="cuda")
        comm.all_gather(x, out)
        torch.cuda.synchronize()
        check(f"allgather n={n}", torch.equal(out, torch.cat([gen(r, n, torch.bfloat16) for r in range(world)])))
        full = gen(rank, n * world, torch.float32, salt=3)
        rs = torch.empty(n, dtype=torch.float32, device="cuda")
        comm.reduce_scatter(full, rs)
        torch.cuda.synchronize()
        check(f"reducescatter n={n}", close(rs, ref_reduce(world, n * world, torch.float32, ReduceOp.SUM, salt=3)[rank * n:(rank + 1) * n], torch.float32, world))
        for root in (0, world - 1):
            b = gen(rank, n, torch.float32, salt=5)
            comm.broadcast(b, root)
            torch.cuda.synchronize()
            check(f"broadcast n={n} root={root}", torch.equal(b, gen(root, n, torch.float32, salt=5)))
            x = gen(rank, n, torch.float32, salt=6)
            out = torch.zeros(n, dtype=torch.float32, device="cuda")
            comm.reduce(x, out, root)
            torch.cuda.synchronize()
            if rank == root:
                check(f"reduce n={n} root={root}", close(out, ref_reduce(world, n, torch.float32, ReduceOp.SUM, salt=6), torch.float32, world))
            send = gen(rank, n * world, torch.float32, salt=7)
            recv = torch.zeros(n, dtype=torch.float32, device="cuda")
            comm.scatter(send, recv, root)
            torch.cuda.synchronize()
            check(f"scatter n={n} root={root}", torch.equal(recv, gen(root, n * world, torch.float32, salt=7)[rank * n:(rank + 1) * n]))
        send = gen(rank, n * world, torch.float32, salt=8)
        recv = torch.zeros(n * world, dtype=torch.float32, device="cuda")
        comm.all_to_all(send, recv)
        torch.cuda.synchronize()
        want = torch.cat([gen(s, n * world, torch.float32, salt=8)[rank * n:(rank + 1) * n] for s in range(world)])
        check(f"alltoall n={n}", torch.equal(recv, want))
    # variable-count gather / reduce-scatter (zero-length contributions included) and unsigned bytes
    vcnt = [((7 * r) % 5) * 1031 for r in range(world)]
    vdis = [sum(vcnt[:r]) for r in range(world)]
    mine = gen(rank, max(1, vcnt[rank]), torch.float32, salt=21)[:vcnt[rank]]
    agv = torch.zeros(max(1, sum(vcnt)), dtype=torch.float32, device="cuda")
    comm.all_gather_v(mine if vcnt[rank] else None, agv, vcnt, vdis)
    torch.cuda.synchronize()
    want = torch.cat([gen(r, max(1, vcnt[r]), torch.float32, salt=21)[:vcnt[r]] for r in range(world)])
    check("allgatherv", torch.equal(agv[:want.numel()], want))
    full = gen(rank, max(1, sum(vcnt)), torch.float32, salt=22)
    rsv = torch.zeros(max(1, vcnt[rank]), dtype=torch.float32, device="cuda")
    comm.reduce_scatter_v(full, vcnt, vdis, rsv if vcnt[rank] else None)
    torch.cuda.synchronize()
    ref = ref_reduce(world, max(1, sum(vcnt)), torch.float32, ReduceOp.SUM, salt=22)
    check("reducescatterv", close(rsv[:vcnt[rank]], ref[vdis[rank]:vdis[rank] + vcnt[rank]], torch.float32, world))
    u8 = (torch.arange(5000, device="cuda") % 7 + rank).to(torch.uint8)
    u8o = torch.empty_like(u8)
    comm.all_reduce(u8, u8o, ReduceOp.MAX)
    torch.cuda.synchronize()
    check("allreduce uint8 max", torch.equal(u8o, (torch.arange(5000, device="cuda") % 7 + world - 1).to(torch.uint8)))
    # CUDA graph capture: all synchronisation state is on the device, so a captured operator replays with new data
    n = 200_000
    gx = gen(rank, n, torch.float32, salt=30)
    gout = torch.empty_like(gx)
    ggat = torch.empty(n * world, dtype=torch.float32, device="cuda")
    comm.all_reduce(gx, gout)
    comm.all_gather(gx, ggat)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        comm.all_reduce(gx, gout)
        comm.all_gather(gout, ggat)
    for it in range(3):
        gx.copy_(gen(rank, n, torch.float32, salt=31 + it))
        graph.replay()
        torch.cuda.synchronize()
        ref = ref_reduce(world, n, torch.float32, ReduceOp.SUM, salt=31 + it)
        check(f"graph replay {it} allreduce", close(gout, ref, torch.float32, world))
        check(f"graph replay {it} allgather", torch.equal(ggat, gout.repeat(world)))
    # eager calls after replays: the device-side sequence numbers moved on during the replays
    comm.all_reduce(gx, gout)
    torch.cuda.synchronize()
    check("eager after graph", close(gout, ref_reduce(world, n, torch.float32, ReduceOp.SUM, salt=33), torch.float32, world))
    # AlltoAllV with a skewed matrix
    M = [[((i * 7 + j * 13) % 5) * 1000 + (i + j) % 2 for j in range(world)] for i in range(world)]
    send = gen(rank, max(1, sum(M[rank])), torch.float32, salt=9)
    recv = torch.zeros(max(1, sum(M[j][rank] for j in range(world))), dtype=torch.float32, device="cuda")
    sd = [sum(M[rank][:j]) for j in range(world)]
    rc = [M[j][rank] for j in range(world)]
    rd = [sum(rc[:j]) for j in range(world)]
    comm.all_to_all_v(send, M[rank], sd, recv, rc, rd)
    torch.cuda.synchronize()
    want = torch.cat([gen(j, max(1, sum(M[j])), torch.float32, salt=9)[sum(M[j][:rank]):sum(M[j][:rank]) + M[j][rank]] for j in range(world)])
    check("alltoallv", torch.equal(recv[:want.numel()], want))
    recv.zero_()
    comm.all_to_all_vc(send, M, recv)
    torch.cuda.synchronize()
    check("alltoallvc", torch.equal(recv[:want.numel()], want))
    # a rank that sends nothing, a rank that receives nothing, one pair above half of the scratch window
    half = (int(os.environ.get("HCCL_BUFFSIZE", "200")) << 20) // 2
    big = half // 4 + 4096                             # fp32 elements: a little more than half of the scratch window
    M = [[1000 * ((i + 2 * j) % 3) + i + 1 for j in range(world)] for i in range(world)]
    M[0][world - 1] = big
    if world > 2:                                      # with two ranks a zero row and a zero column would leave nothing to move
        for j in range(world):
            M[1][j] = 0
            M[j][2 if world > 3 else 1] = 0
    else:
        M[1] = [0, 0]
    send = gen(rank, max(1, sum(M[rank])), torch.float32, salt=19)
    rc = [M[j][rank] for j in range(world)]
    recv = torch.full((max(1, sum(rc)),), -3.0, dtype=torch.float32, device="cuda")
    comm.all_to_all_v(send, M[rank], [sum(M[rank][:j]) for j in range(world)], recv, rc, [sum(rc[:j]) for j in range(world)])
    torch.cuda.synchronize()
    parts = [gen(j, max(1, sum(M[j])), torch.float32, salt=19)[sum(M[j][:rank]):sum(M[j][:rank]) + M[j][rank]] for j in range(world)]
    want = torch.cat(parts)
    check("alltoallv zero row / column / large pair", torch.equal(recv[:want.numel()], want) and bool(torch.all(recv[want.numel():] == -3.0)))
    recv.fill_(-3.0)
    comm.all_to_all_vc(send, M, recv)
    torch.cuda.synchronize()
    check("alltoallvc zero row / column / large pair", torch.equal(recv[:want.numel()], want))
    del send, recv, parts, want
    # send / recv ring, then batch
    n = 700_000
    x = gen(rank, n, torch.float32, salt=11)
    y = torch.zeros(n, dtype=torch.float32, device="cuda")
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    if rank % 2 == 0:
        comm.send(x, nxt)
        comm.recv(y, prv)
    else:
        comm.recv(y, prv)
        comm.send(x, nxt)
    torch.cuda.synchronize()
    check("send/recv ring", torch.equal(y, gen(prv, n, torch.float32, salt=11)))
    y.zero_()
    comm.batch_send_recv([("send", x, nxt), ("recv", y, prv)])
    torch.cuda.synchronize()
    check("batch_send_recv ring", torch.equal(y, gen(prv, n, torch.float32, salt=11)))
    # zero-copy on registered windows: symmetric allocations at the same heap offset on every rank; from 1 MB up the selector
    # takes the kernels that read / write the windows directly (through the switch when the multicast mapping exists)
    zn = 1 << 20                                              # 4 MB of fp32
    # an explicit engine or algorithm request wins over the zero-copy rule
    expect_zc = "HCCL_OP_EXPANSION_MODE" not in os.environ and "HCCL_ALGO_NAME" not in os.environ
    zc_ok = lambda suffix: comm.last_algorithm().endswith(suffix) == expect_zc    # noqa: E731
    win_in = comm.sym_tensor(zn * world, torch.float32)
    win_out = comm.sym_tensor(zn * world, torch.float32)
    for it in range(2):
        win_in[:zn].copy_(gen(rank, zn, torch.float32, salt=40 + it))
        comm.all_reduce(win_in[:zn], win_out[:zn])
        torch.cuda.synchronize()
        check(f"zero-copy allreduce selected ({comm.last_algorithm()})", zc_ok("AllReduceZeroCopy"))
        check(f"zero-copy allreduce it={it}", close(win_out[:zn], ref_reduce(world, zn, torch.float32, ReduceOp.SUM, salt=40 + it), torch.float32, world))
    comm.all_reduce(win_in[:zn])                              # in place
    torch.cuda.synchronize()
    check("zero-copy allreduce in place", close(win_in[:zn], ref_reduce(world, zn, torch.float32, ReduceOp.SUM, salt=41), torch.float32, world))
    win_in.copy_(gen(rank, zn * world, torch.float32, salt=43))
    rs_out = torch.empty(zn, dtype=torch.float32, device="cuda")
    comm.reduce_scatter(win_in, rs_out)
    torch.cuda.synchronize()
    check(f"zero-copy reducescatter selected ({comm.last_algorithm()})", zc_ok("ReduceScatterZeroCopy"))
    check("zero-copy reducescatter", close(rs_out, ref_reduce(world, zn * world, torch.float32, ReduceOp.SUM, salt=43)[rank * zn:(rank + 1) * zn], torch.float32, world))
    ag_in = gen(rank, zn, torch.float32, salt=44)
    comm.all_gather(ag_in, win_out)
    torch.cuda.synchronize()
    check(f"zero-copy allgather selected ({comm.last_algorithm()})", zc_ok("AllGatherZeroCopy"))
    check("zero-copy allgather", torch.equal(win_out, torch.cat([gen(r, zn, torch.float32, salt=44) for r in range(world)])))
    win_out[:zn].copy_(gen(rank, zn, torch.float32, salt=45))
    comm.broadcast(win_out[:zn], world - 1)
    torch.cuda.synchronize()
    check(f"zero-copy broadcast selected ({comm.last_algorithm()})", zc_ok("BroadcastZeroCopy"))
    check("zero-copy broadcast", torch.equal(win_out[:zn], gen(world - 1, zn, torch.float32, salt=45)))
    # small payloads and unregistered buffers keep the staged kernels
    comm.all_reduce(win_in[:1024], win_out[:1024])
    torch.cuda.synchronize()
    check("small payload stays staged", not comm.last_algorithm().endswith("ZeroCopy"))
    comm.sym_free(win_out)
    comm.sym_free(win_in)
    # tensors from a torch memory pool whose segments are registered blocks of the heap: plain torch code, zero-copy kernels
    pool = comm.mem_pool()
    with torch.cuda.use_mem_pool(pool):
        pg_in = torch.empty(zn, dtype=torch.float32, device="cuda")
        pg_out = torch.empty(zn, dtype=torch.float32, device="cuda")
    pg_in.copy_(gen(rank, zn, torch.float32, salt=47))
    comm.all_reduce(pg_in, pg_out)
    torch.cuda.synchronize()
    check(f"pool tensors are registered windows ({comm.last_algorithm()})", zc_ok("AllReduceZeroCopy"))
    check("pool tensors allreduce", close(pg_out, ref_reduce(world, zn, torch.float32, ReduceOp.SUM, salt=47), torch.float32, world))
    del pg_in, pg_out
    del pool                                                  # segments go back to the heap through the free hook
    comm.barrier()
    torch.cuda.synchronize()
    check("async error clean", comm.async_error() == 0)
    comm.destroy()
    if fails:
        print(f"[rank {rank}] {len(fails)} failures: {fails[:8]}", flush=True)
        sys.exit(1)
    if rank == 0:
        print(f"all multi-GPU collective checks passed on {world} ranks (nvls={os.environ.get('HCCL_NVLS_ENABLE', 'auto')}, "
              f"engine={os.environ.get('HCCL_OP_EXPANSION_MODE', 'auto')}, buffsize={os.environ.get('HCCL_BUFFSIZE', 'default')})", flush=True)


if __name__ == "__main__":
    main()
