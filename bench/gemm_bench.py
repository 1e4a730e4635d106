#!/usr/bin/env python
"""Single-GPU throughput of the tcgen05 GEMM against cuBLAS (torch.matmul) on the tensor-parallel
MLP shapes (Llama-3-70B, TP=8: d=8192, ffn/8=3584, 8192 tokens).  CUDA-event timing, L2 flushed
between iterations, fraction of the measured cuBLAS peak from MEASURED_PEAKS.json.

Reference parity: none -- the reference has no GEMM; cuBLAS is the baseline.
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200.ops import gemm_bf16  # noqa: E402


def time_interleaved(fns, iters=30, warmup=3):
    """Times several implementations of one problem turn by turn (so that clock and power state
    hit them alike); returns {name: (median_ms, best_ms)}."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        for fn in fns.values():
            fn()
    torch.cuda.synchronize()
    times = {k: [] for k in fns}
    for _ in range(iters):
        for name, fn in fns.items():
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times[name].append(s.elapsed_time(e))
    return {k: (statistics.median(v), min(v)) for k, v in times.items()}


def grouped_bench(args, peak):
    """The expert FFN of one expert-parallel rank (BASELINE config 5: 64 experts over 8 ranks, top-8 of
    N(0,1) logits, d=4096, expert FFN 1536, 16384 tokens per rank): two grouped GEMMs."""
    import torch.nn.functional as F
    from asystem_amem_b200.ops import grouped_gemm_bf16, interleave_gate_up
    El, d, ffn, rows = 8, 4096, 1536, 16384 * 8
    g = torch.Generator().manual_seed(0)
    counts = torch.multinomial(torch.ones(El), rows, replacement=True, generator=g).bincount(minlength=El)
    offs = torch.zeros(El + 1, dtype=torch.int32)
    offs[1:] = counts.cumsum(0)
    offs_dev = offs.cuda()
    x = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(El, 2 * ffn, d, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(El, d, ffn, device="cuda") * 0.02).to(torch.bfloat16)
    w13i = interleave_gate_up(w13, ffn)
    act = torch.empty(rows, ffn, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)

    def ours():
        grouped_gemm_bf16(x, w13i, offs_dev, out=act, rows_hint=rows, swiglu=True)
        grouped_gemm_bf16(act, w2, offs_dev, out=y, rows_hint=rows)

    def loop():
        o = offs_dev.tolist()                         # the host synchronisation a per-expert loop needs
        for e in range(El):
            h = x[o[e]:o[e + 1]] @ w13[e].t()
            a = (F.silu(h[:, :ffn].float()) * h[:, ffn:].float()).to(torch.bfloat16)
            torch.matmul(a, w2[e].t(), out=y[o[e]:o[e + 1]])

    t = time_interleaved({"amem": ours, "cublas_loop": loop}, iters=args.iters)
    fl = 2.0 * rows * d * (3 * ffn)
    row = {"case": "moe expert FFN of one rank, 2 grouped GEMMs (SwiGLU in the first epilogue)", "rows": rows, "experts": El, "d": d, "ffn": ffn,
           "amem_ms": round(t["amem"][0], 4), "cublas_loop_ms": round(t["cublas_loop"][0], 4),
           "amem_tflops": round(fl / t["amem"][0] / 1e9, 1), "frac_of_measured_peak": round(fl / t["amem"][0] / 1e9 / peak, 3),
           "vs_cublas_loop": round(t["cublas_loop"][0] / t["amem"][0], 3)}
    print(json.dumps(row), flush=True)
    with open(args.out, "a") as f:
        f.write(json.dumps(row) + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bench_results/gemm.jsonl")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--grouped", action="store_true",
                    help="time the grouped GEMM (MoE expert FFN of one rank: 8 experts, d=4096, ffn=1536, 16384 x 8 routed rows) "
                         "against a per-expert loop of cuBLAS calls that reads the group boundaries on the host")
    ap.add_argument("--shapes", default="8192x3584x8192,8192x8192x3584,8192x8192x8192,4096x4096x4096,1024x3584x8192,2048x2048x2048")
    args = ap.parse_args()
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    peak = peaks.get("bf16_tflops", 1590.0)
    shapes = [tuple(int(v) for v in sh.split("x")) for sh in args.shapes.split(",")]
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    if args.grouped:
        grouped_bench(args, peak)
        return
    with open(args.out, "w") as f:
        for M, N, K in shapes:
            a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            b = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

            def ours(split):
                def run():
                    os.environ["AMEM_GEMM_SPLITK"] = split
                    gemm_bf16(a, b, out)
                return run

            t = time_interleaved({"amem": ours("1"), "amem_nosplit": ours("0"), "cublas": lambda: torch.matmul(a, b.t(), out=out)},
                                 iters=args.iters)
            os.environ["AMEM_GEMM_SPLITK"] = "1"
            fl = 2.0 * M * N * K
            med, best = t["amem"]
            row = {"M": M, "N": N, "K": K, "amem_ms": round(med, 4), "amem_best_ms": round(best, 4),
                   "amem_no_tail_split_ms": round(t["amem_nosplit"][0], 4),
                   "cublas_ms": round(t["cublas"][0], 4), "cublas_best_ms": round(t["cublas"][1], 4),
                   "amem_tflops": round(fl / med / 1e9, 1), "cublas_tflops": round(fl / t["cublas"][0] / 1e9, 1),
                   "frac_of_measured_peak": round(fl / med / 1e9 / peak, 3), "vs_cublas": round(t["cublas"][0] / med, 3),
                   "timing": "median of %d, L2 flushed before every launch, implementations interleaved" % args.iters}
            print(json.dumps(row), flush=True)
            f.write(json.dumps(row) + "\n")


if __name__ == "__main__":
    main()
