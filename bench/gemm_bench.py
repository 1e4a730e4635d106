#!/usr/bin/env python
"""Single-GPU throughput of the tcgen05 GEMM against cuBLAS (torch.matmul) on the tensor-parallel
MLP shapes (Llama-3-70B, TP=8: d=8192, ffn/8=3584, 8192 tokens).  CUDA-event timing, L2 flushed
between iterations, fraction of the measured cuBLAS peak from MEASURED_PEAKS.json."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200.ops import gemm_bf16  # noqa: E402


def time_fn(fn, iters=10, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    best, total = 1e9, 0.0
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e)
        best = min(best, ms)
        total += ms
    return best, total / iters


def main():
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    peak = peaks.get("bf16_tflops", 1590.0)
    shapes = [(8192, 3584, 8192), (8192, 8192, 3584), (8192, 8192, 8192), (4096, 4096, 4096), (1024, 3584, 8192)]
    rows = []
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ours_best, ours_mean = time_fn(lambda: gemm_bf16(a, b, out))
        ref_best, ref_mean = time_fn(lambda: torch.matmul(a, b.t(), out=out))
        fl = 2.0 * M * N * K
        rows.append({"M": M, "N": N, "K": K, "amem_ms": round(ours_best, 4), "cublas_ms": round(ref_best, 4),
                     "amem_tflops": round(fl / ours_best / 1e9, 1), "cublas_tflops": round(fl / ref_best / 1e9, 1),
                     "frac_of_measured_peak": round(fl / ours_best / 1e9 / peak, 3),
                     "vs_cublas": round(ref_best / ours_best, 3)})
        print(json.dumps(rows[-1]), flush=True)


if __name__ == "__main__":
    main()
