"""MoE expert-parallel dispatch/combine: fused kernels of this library against NCCL all-to-all + torch permute/weighted-sum.

Launch with torchrun (one process per GPU). DeepSeek-V3-like defaults: hidden 7168, 256 experts, top-8, 4096 tokens per rank;
router logits N(0,1) plus a Zipf(s=1.1)-shaped per-expert bias; tokens N(0,1). Checks the fused result against the baseline
result, then reports device time (CUDA events, max over ranks) for dispatch + combine with identity experts.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--mxfp8", action="store_true")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    os.environ.setdefault("HCCL_SYM_HEAP_MB", "6144")
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from hccl_b200.comm import init_from_env
    from hccl_b200.ops.moe import MoeDispatcher
    comm = init_from_env()
    rank, n = comm.rank, comm.size
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    EL = E // n
    g = torch.Generator(device="cuda").manual_seed(4242 + rank)
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    gb = torch.Generator(device="cuda").manual_seed(7)
    perm = torch.randperm(E, generator=gb, device="cuda")
    bias = torch.empty(E, device="cuda")
    bias[perm] = (1.0 / torch.arange(1, E + 1, device="cuda").float() ** 1.1)
    bias = (bias / bias.max()) * 3.0      # the most popular expert gets +3 on its logit
    logits = torch.randn(T, E, generator=g, device="cuda") + bias
    topv, topi = torch.topk(logits, K, dim=1)
    weights = torch.softmax(topv, dim=1).float().contiguous()
    idx = topi.to(torch.int32).contiguous()
    cap = int(2.5 * T * K)
    disp = MoeDispatcher(comm, E, K, H, T, max_recv_rows=cap, mxfp8=args.mxfp8)

    def fused():
        recv_x, recv_scales, counts, src = disp.dispatch(x, idx)
        if not args.mxfp8:
            rows = min(cap, T * K * 2)
            disp.expert_out[:rows].copy_(recv_x[:rows])          # identity experts
        return disp.combine(weights)

    def fused_comm_only():
        disp.dispatch(x, idx)
        return disp.combine(weights)

    # ---- baseline: sort by destination expert, NCCL all_to_all_single both ways, weighted sum
    flat_e = idx.flatten().long()
    order = torch.argsort(flat_e, stable=True)
    send_counts_e = torch.bincount(flat_e, minlength=E)
    in_splits = send_counts_e.view(n, EL).sum(1)
    out_splits_t = torch.empty_like(in_splits)
    dist.all_to_all_single(out_splits_t, in_splits)
    in_sp, out_sp = in_splits.tolist(), out_splits_t.tolist()
    tok_of = torch.arange(T, device="cuda").repeat_interleave(K)

    def baseline():
        send = x[tok_of[order]]
        recv = torch.empty(sum(out_sp), H, dtype=torch.bfloat16, device="cuda")
        dist.all_to_all_single(recv, send, out_sp, in_sp)
        back = torch.empty_like(send)
        dist.all_to_all_single(back, recv, in_sp, out_sp)          # identity experts
        contrib = torch.empty(T * K, H, dtype=torch.bfloat16, device="cuda")
        contrib[order] = back
        return (contrib.view(T, K, H).float() * weights.unsqueeze(-1)).sum(1).to(torch.bfloat16)

    # MXFP8 dispatch baseline: a separate quantisation pass (1 x 32 blocks, e8m0 scales, OCP rule) written with torch ops, payload and
    # scales in two all-to-alls, bf16 on the way back (the experts' output stands in as a persistent bf16 buffer, as on the fused side)
    HB = H // 32
    back_src = torch.zeros(sum(out_sp), H, dtype=torch.bfloat16, device="cuda")

    def baseline_mx():
        send = x[tok_of[order]]
        v = send.float().view(-1, HB, 32)
        e = (v.abs().amax(dim=2).view(torch.int32) >> 23) & 0xFF
        se = (e - 8).clamp(0, 254)
        inv = ((254 - se) << 23).to(torch.int32).view(torch.float32)
        q = (v * inv.unsqueeze(2)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).view(-1, H)
        sc = se.to(torch.uint8)
        recv_q = torch.empty(sum(out_sp), H, dtype=torch.uint8, device="cuda")
        recv_s = torch.empty(sum(out_sp), HB, dtype=torch.uint8, device="cuda")
        dist.all_to_all_single(recv_q, q, out_sp, in_sp)
        dist.all_to_all_single(recv_s, sc, out_sp, in_sp)
        back = torch.empty_like(send)
        dist.all_to_all_single(back, back_src, in_sp, out_sp)
        contrib = torch.empty(T * K, H, dtype=torch.bfloat16, device="cuda")
        contrib[order] = back
        return (contrib.view(T, K, H).float() * weights.unsqueeze(-1)).sum(1).to(torch.bfloat16)

    def timed(f, it):
        for _ in range(3):
            f()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(it):
            f()
        e.record(); torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / it], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    ok = True
    if not args.mxfp8:
        a, b = fused(), baseline()
        torch.cuda.synchronize()
        err = (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)
        ok = err < 2e-2
        if not ok:
            print(f"[rank {rank}] MISMATCH fused vs baseline: rel err {err}", flush=True)
    t_f = timed(fused_comm_only, args.iters)
    t_b = timed(baseline_mx if args.mxfp8 else baseline, args.iters)
    out_bytes = (1 + 1 / 32) if args.mxfp8 else 2                       # dispatch: e4m3 + one scale byte per 32, or bf16
    moved = T * K * H * (out_bytes + 2) * (n - 1) / n                   # bytes leaving + returning per rank (uniform-routing estimate)
    load = torch.tensor([float(sum(out_sp))], device="cuda")
    dist.all_reduce(load, op=dist.ReduceOp.MAX)
    if rank == 0:
        res = dict(ranks=n, tokens=T, hidden=H, experts=E, topk=K, mxfp8=args.mxfp8, fused_ms=round(t_f, 4), nccl_torch_ms=round(t_b, 4),
                   speedup=round(t_b / t_f, 3), fused_GBs_per_rank=round(moved / (t_f * 1e-3) / 1e9, 1), results_match=ok,
                   routing="N(0,1) logits + Zipf(1.1)-shaped expert bias", busiest_rank_rows_over_mean=round(load.item() / (T * K), 3))
        print(json.dumps(res), flush=True)
        if args.json:
            with open(args.json, "w") as f:
                json.dump(res, f)
    disp.close()
    comm.destroy()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
