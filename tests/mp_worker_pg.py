"""Worker for the torch.distributed backend tests (CPU tensors -> host simulation backend; CUDA tensors when available)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
import hccl_b200.parallel  # noqa: E402,F401  (registers "hccl")


def main():
    use_cuda = os.environ.get("PG_DEVICE", "cpu") == "cuda"
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda") if use_cuda else torch.device("cpu")
    dist.init_process_group("hccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    x = torch.full((1000,), float(rank + 1), device=dev)
    dist.all_reduce(x)
    assert torch.all(x == world * (world + 1) / 2)
    y = torch.arange(8, dtype=torch.float32, device=dev) + rank
    dist.all_reduce(y, op=dist.ReduceOp.MAX)
    assert torch.equal(y, torch.arange(8, dtype=torch.float32, device=dev) + world - 1)
    b = torch.full((17,), float(rank), device=dev)
    dist.broadcast(b, src=world - 1)
    assert torch.all(b == world - 1)
    outs = [torch.zeros(5, device=dev) for _ in range(world)]
    dist.all_gather(outs, torch.full((5,), float(rank), device=dev))
    assert all(torch.all(outs[r] == r) for r in range(world))
    big = torch.zeros(world * 6, device=dev)
    dist.all_gather_into_tensor(big, torch.full((6,), float(rank), device=dev))
    assert all(torch.all(big[r * 6:(r + 1) * 6] == r) for r in range(world))
    rs = torch.zeros(4, device=dev)
    dist.reduce_scatter_tensor(rs, torch.arange(world * 4, dtype=torch.float32, device=dev))
    assert torch.equal(rs, world * torch.arange(rank * 4, rank * 4 + 4, dtype=torch.float32, device=dev))
    a2a_in = torch.arange(world * 3, dtype=torch.float32, device=dev) + 100 * rank
    a2a_out = torch.zeros(world * 3, device=dev)
    dist.all_to_all_single(a2a_out, a2a_in)
    want = torch.cat([torch.arange(rank * 3, rank * 3 + 3, dtype=torch.float32, device=dev) + 100 * s for s in range(world)])
    assert torch.equal(a2a_out, want)
    # uneven all_to_all_single
    in_splits = [(rank + j) % 3 + 1 for j in range(world)]
    out_splits = [(s + rank) % 3 + 1 for s in range(world)]
    src = torch.full((sum(in_splits), 2), float(rank), device=dev)
    dst = torch.zeros(sum(out_splits), 2, device=dev)
    dist.all_to_all_single(dst, src, out_splits, in_splits)
    off = 0
    for s in range(world):
        assert torch.all(dst[off:off + out_splits[s]] == s)
        off += out_splits[s]
    r = torch.full((9,), float(rank + 1), device=dev)
    dist.reduce(r, dst=0)
    if rank == 0:
        assert torch.all(r == world * (world + 1) / 2)
    if world >= 2:
        if rank == 0:
            dist.send(torch.full((11,), 7.0, device=dev), dst=1)
        elif rank == 1:
            t = torch.zeros(11, device=dev)
            dist.recv(t, src=0)
            assert torch.all(t == 7.0)
    dist.barrier()
    # DistributedDataParallel: bucketed gradient all-reduce through the backend, overlapped with backward
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).to(dev)
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index] if use_cuda and dev.index is not None else None, bucket_cap_mb=0.01)
    torch.manual_seed(100 + rank)
    inp = torch.randn(16, 32, device=dev)
    ddp(inp).sum().backward()
    g = model[0].weight.grad.clone()
    gs = [torch.zeros_like(g) for _ in range(world)]
    dist.all_gather(gs, g)
    assert all(torch.allclose(gs[0], gi, atol=1e-6) for gi in gs), "DDP gradients differ across ranks"
    if use_cuda and world > 1:
        # tensors from the memory pool over registered blocks of the group's communicator: the all-reduce runs on the window directly
        import ctypes

        from hccl_b200._lib import lib
        from hccl_b200.parallel import process_group as hpg
        pool = hpg.mem_pool()
        with torch.cuda.use_mem_pool(pool):
            big = torch.full((1 << 20,), float(rank + 1), device=dev)
        dist.all_reduce(big)
        torch.cuda.synchronize()
        assert torch.all(big == world * (world + 1) / 2)

        class Rec(ctypes.Structure):
            _fields_ = [("seq", ctypes.c_uint64), ("opType", ctypes.c_uint32), ("dataType", ctypes.c_uint32), ("reduceOp", ctypes.c_uint32),
                        ("root", ctypes.c_uint32), ("engine", ctypes.c_uint32), ("pad", ctypes.c_uint32), ("count", ctypes.c_uint64),
                        ("algName", ctypes.c_char * 64), ("beginNs", ctypes.c_uint64), ("endNs", ctypes.c_uint64)]
        h, recs, cnt = ctypes.c_void_p(), (Rec * 1)(), ctypes.c_uint32()
        assert lib().HcclGetAllocatorComm(ctypes.byref(h)) == 0 and h.value
        assert lib().HcclGetLastOps(h, recs, 1, ctypes.byref(cnt)) == 0 and cnt.value == 1
        alg = recs[0].algName.decode()
        assert alg.endswith("ZeroCopy") or "HCCL_ZERO_COPY" in os.environ or "HCCL_ALGO_NAME" in os.environ, alg
        if rank == 0:
            print(f"pool tensor all-reduce ran {alg}", flush=True)
        del big, pool
    if use_cuda:
        torch.cuda.synchronize()
    dist.destroy_process_group()
    if rank == 0:
        print(f"process group checks passed ({dev.type}, world {world})", flush=True)


if __name__ == "__main__":
    main()
