#!/usr/bin/env python
"""Tensor-parallel MLP block, Llama-3-70B shape (d=8192, ffn=28672, 8192 tokens, bf16, weights
N(0, 0.02)): the fused all-gather->GEMM and GEMM->reduce-scatter kernels against cuBLAS + NCCL
back to back, with the communicator paused and resumed between the 20 iterations.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29530 bench/tp_mlp.py

Times are CUDA events on the launching stream, max over ranks.  Roofline per fused kernel: the
slower of FLOPs / measured cuBLAS peak and NVLink bytes / 770 GB/s (measured peer copy rate).

Reference parity: none -- baseline is what the reference's users run, cuBLAS + NCCL back to
back.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator, pause_all, resume_all  # noqa: E402
from asystem_amem_b200.ops import all_gather_gemm, gemm_reduce_scatter  # noqa: E402
from asystem_amem_b200.utils import load_measured_peaks  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-pause", action="store_true", help="do not pause/resume between iterations")
    ap.add_argument("--out", default="bench_results/tp_mlp.jsonl")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    dist.all_reduce(torch.zeros(1, device="cuda"))
    gloo = dist.new_group(backend="gloo")
    comm = Communicator.from_torch_distributed(gloo)
    peaks = load_measured_peaks()
    M, D, Fl = args.tokens, args.dim, args.ffn // world
    rows = M // world
    g = torch.Generator(device="cuda").manual_seed(rank)
    x_shard = torch.randn(rows, D, device="cuda", generator=g).to(torch.bfloat16)
    w1 = (torch.randn(Fl, D, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(D, Fl, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    h = torch.empty(M, Fl, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(rows, D, device="cuda", dtype=torch.bfloat16)
    x_full = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    y_full = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    align = torch.zeros(8, device="cuda")

    def fused_ag():
        all_gather_gemm(comm, x_shard, w1, out=h)

    def fused_rs():
        gemm_reduce_scatter(comm, h, w2, out=y)

    def base_ag():
        dist.all_gather_into_tensor(x_full, x_shard)
        torch.matmul(x_full, w1.t(), out=h)

    def base_rs():
        torch.matmul(h, w2.t(), out=y_full)
        dist.reduce_scatter_tensor(y, y_full)

    def timed(fn, pause_between):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier(group=gloo)
        tot = 0.0
        for _ in range(args.iters):
            flush.zero_()
            comm.all_reduce(align)   # ranks leave resume at different moments: line the streams up on the device
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            tot += s.elapsed_time(e)
            if pause_between:
                pause_all()
                resume_all()
        t = torch.tensor([tot / args.iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return float(t.item())

    res = {"n_gpus": world, "tokens": M, "dim": D, "ffn_local": Fl}
    res["paused_between_iterations"] = not args.no_pause
    res["ag_gemm_fused_ms"] = timed(fused_ag, not args.no_pause)
    res["ag_gemm_cublas_nccl_ms"] = timed(base_ag, False)
    res["gemm_rs_fused_ms"] = timed(fused_rs, not args.no_pause)
    res["gemm_rs_cublas_nccl_ms"] = timed(base_rs, False)
    flops = 2.0 * M * Fl * D
    t_compute = flops / (peaks["bf16_tflops"] * 1e12) * 1e3
    link = 770e9
    ag_bytes = (world - 1) * rows * D * 2          # received per rank
    rs_bytes = (world - 1) * rows * D * 2          # sent per rank (bf16 partials)
    res["roofline_ms_ag"] = max(t_compute, ag_bytes / link * 1e3)
    res["roofline_ms_rs"] = max(t_compute, rs_bytes / link * 1e3)
    res["ag_frac_of_roofline"] = res["roofline_ms_ag"] / res["ag_gemm_fused_ms"]
    res["rs_frac_of_roofline"] = res["roofline_ms_rs"] / res["gemm_rs_fused_ms"]
    res["ag_speedup_vs_cublas_nccl"] = res["ag_gemm_cublas_nccl_ms"] / res["ag_gemm_fused_ms"]
    res["rs_speedup_vs_cublas_nccl"] = res["gemm_rs_cublas_nccl_ms"] / res["gemm_rs_fused_ms"]
    res["peaks"] = peaks.get("source")
    # which schedule the all-gather -> GEMM kernel ran (host arithmetic of the library)
    import ctypes
    from asystem_amem_b200.bindings import load_library
    sched, per_flag = ctypes.c_int(), ctypes.c_int()
    if load_library().amemAllGatherGemmPlan(world, rows, D, ctypes.byref(sched), ctypes.byref(per_flag), None) == 0:
        res["ag_schedule"] = "mover warps in every CTA" if sched.value else "dedicated mover CTAs"
        res["ag_rows_per_ready_flag"] = per_flag.value
    # numerics of the fused kernels against the library path
    base_ag()
    ref_h = h.clone()
    fused_ag()
    torch.cuda.synchronize()
    res["ag_max_abs_diff_vs_cublas"] = float((h.float() - ref_h.float()).abs().max())
    res["device_errors"] = comm.async_error()
    if rank == 0:
        res = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items()}
        print(json.dumps(res), flush=True)
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "a") as f:
            f.write(json.dumps(res) + "\n")
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
