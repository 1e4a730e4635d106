#!/usr/bin/env python
"""Hybrid-parallel MoE layer with split communicators (TP=2 x EP=world/2 through ncclCommSplit):
64 experts, top-8 routing from N(0,1) logits, d=4096, expert FFN 1536, 16384 tokens per rank,
bf16.  Measures the fused dispatch and combine against torch index_select + NCCL all-to-all,
then pauses and resumes ALL communicators together for --cycles cycles, checking that the
layer's output stays bit-identical and that device memory use is flat.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29540 bench/moe.py --cycles 100

Reference parity: the reference names all-to-all as the largest consumer of NCCL memory
(README.md:132, docs/images/result1.webp) and pauses every communicator of the process together
(nccl_patch/nccl_2.27.5-1.diff:70-77).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator, pause_all, resume_all  # noqa: E402
from asystem_amem_b200.models import MoELayer  # noqa: E402
from asystem_amem_b200.parallel import make_grid  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=1536)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--cycles", type=int, default=100)
    ap.add_argument("--out", default="bench_results/moe.jsonl")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    dist.all_reduce(torch.zeros(1, device="cuda"))
    gloo = dist.new_group(backend="gloo")
    world_comm = Communicator.from_torch_distributed(gloo)
    tp = args.tp if world % args.tp == 0 and world > 1 else 1
    tp_comm, ep_comm = make_grid(world_comm, tp)
    ep_ranks = [r for r in range(world) if r % tp == rank % tp]
    ep_group = None
    for pos in range(tp):  # every rank must take part in every new_group call
        grp = dist.new_group([r for r in range(world) if r % tp == pos])
        if pos == rank % tp:
            ep_group = grp
    n_ep = ep_comm.nranks
    T, D, E, K = args.tokens, args.dim, args.experts, args.topk
    layer = MoELayer(ep_comm, D, args.ffn, E, K, tokens_per_rank=T, capacity_factor=2.0, seed=3)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(T, D, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    top = logits.topk(K, dim=1)
    idx, w = top.indices.to(torch.int32), torch.softmax(top.values, dim=1)
    disp = layer.dispatcher
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier(group=gloo)
        tot = 0.0
        for _ in range(iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            tot += s.elapsed_time(e)
        t = torch.tensor([tot / iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return float(t.item())

    state = {}

    def fused_dispatch():
        state["res"] = disp.dispatch(x, idx)

    def fused_combine():
        disp.combine(idx, w, state["res"].send_pos)

    # baseline: sort pairs by expert, exchange counts, all_to_all_single of the rows, and back
    El = E // n_ep
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    send_rows_idx = order // K
    counts = torch.bincount(flat, minlength=E).view(n_ep, El).sum(1)
    in_splits = counts.tolist()
    out_counts = torch.empty_like(counts)
    dist.all_to_all_single(out_counts, counts, group=ep_group)
    out_splits = out_counts.tolist()
    recv_base = torch.empty(sum(out_splits), D, device="cuda", dtype=torch.bfloat16)
    back = torch.empty(T * K, D, device="cuda", dtype=torch.bfloat16)

    def base_dispatch():
        send = x.index_select(0, send_rows_idx)
        dist.all_to_all_single(recv_base, send, out_splits, in_splits, group=ep_group)

    def base_combine():
        dist.all_to_all_single(back, recv_base, in_splits, out_splits, group=ep_group)
        un = torch.empty_like(back)
        un[order] = back
        return (un.view(T, K, D).float() * w.unsqueeze(2)).sum(1).to(torch.bfloat16)

    res = {"n_gpus": world, "tp": tp, "ep": n_ep, "tokens_per_rank": T, "dim": D, "experts": E, "topk": K}
    res["dispatch_fused_ms"] = timed(fused_dispatch)
    torch.cuda.synchronize()
    total = int(state["res"].expert_offsets[-1])
    disp.y[:total] = state["res"].recv_x[:total]
    res["combine_fused_ms"] = timed(fused_combine)
    res["dispatch_torch_nccl_ms"] = timed(base_dispatch)
    res["combine_torch_nccl_ms"] = timed(base_combine)
    row_bytes = D * 2
    remote = T * K * (n_ep - 1) / n_ep * row_bytes
    res["dispatch_link_gbs"] = remote / (res["dispatch_fused_ms"] * 1e-3) / 1e9
    res["combine_link_gbs"] = remote / (res["combine_fused_ms"] * 1e-3) / 1e9
    res["dispatch_frac_of_770"] = res["dispatch_link_gbs"] / 770.0
    res["combine_frac_of_770"] = res["combine_link_gbs"] / 770.0

    # the whole layer without gradients: routing, dispatch, two grouped tcgen05 GEMMs over all local
    # experts (group boundaries stay on the device), combine; against the same layer with the experts
    # as a per-expert loop of cuBLAS calls that reads the boundaries on the host
    import torch.nn.functional as F
    import time

    def layer_fused():
        with torch.no_grad():
            layer(x)

    def layer_loop():
        with torch.no_grad():
            lg = (x @ layer.router.t()).float()
            tp_ = lg.topk(K, dim=1)
            li, lw = tp_.indices.to(torch.int32), torch.softmax(tp_.values, dim=1)
            r_ = disp.dispatch(x, li)
            offs = r_.expert_offsets.tolist()
            for el in range(layer.El):
                lo, hi = offs[el], offs[el + 1]
                if hi > lo:
                    h = r_.recv_x[lo:hi] @ layer.w13[el].t()
                    a_ = (F.silu(h[:, : args.ffn].float()) * h[:, args.ffn:].float()).to(torch.bfloat16)
                    disp.y[lo:hi] = a_ @ layer.w2[el].t()
            disp.combine(li, lw, r_.send_pos)

    res["layer_forward_fused_ms"] = timed(layer_fused, iters=5)
    res["layer_forward_expert_loop_ms"] = timed(layer_loop, iters=5)
    # all communicators paused and resumed together
    with torch.no_grad():
        first = layer(x).clone()
    torch.cuda.synchronize()
    dist.barrier(group=gloo)
    used0 = torch.cuda.mem_get_info()[0]
    same, drift, freed = True, 0, 0
    cycle_ms = []
    for c in range(args.cycles):
        t0 = time.perf_counter()
        pause_all()
        t1 = time.perf_counter()
        freed = torch.cuda.mem_get_info()[0] - used0
        t2 = time.perf_counter()
        resume_all()
        cycle_ms.append((t1 - t0 + time.perf_counter() - t2) * 1e3)
        if c % 10 == 9 or c == args.cycles - 1:
            with torch.no_grad():
                out = layer(x)
            torch.cuda.synchronize()
            same = same and torch.equal(out, first)
        drift = max(drift, abs(torch.cuda.mem_get_info()[0] - used0))
    flag = torch.tensor([1 if same else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=gloo)
    cyc = torch.tensor(cycle_ms, dtype=torch.float64)
    dist.all_reduce(cyc, op=dist.ReduceOp.MAX, group=gloo)
    res["pause_resume_all_comms_median_ms"] = float(cyc.median())    # world + TP + EP communicators in ONE engine pass
    res["cycles"] = args.cycles
    res["bitwise_equal_after_cycles"] = bool(flag.item())
    res["gib_freed_per_gpu_on_pause"] = freed / 2**30
    res["memory_drift_mib"] = drift / 2**20
    res["device_errors"] = world_comm.async_error() + ep_comm.async_error() + (tp_comm.async_error() if tp_comm else 0)
    if rank == 0:
        res = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items()}
        print(json.dumps(res), flush=True)
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "a") as f:
            f.write(json.dumps(res) + "\n")
    dist.barrier(group=gloo)
    for c in (ep_comm, tp_comm, world_comm):
        if c is not None:
            c.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
