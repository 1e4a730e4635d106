#!/usr/bin/env python
"""Small single-GPU workloads for profiler captures (one kernel family per --case).

Each case launches its kernel a handful of times on inputs larger than the 126 MB L2 but well
under a few GB, so that `ncu --set full -k regex:<kernel> -c 1..3` finishes in a minute or two.
Multi-rank kernels run as emulated ranks (threads of this process, one cooperative grid).

    python bench/ncu_cases.py --case gemm
    ncu --set full --clock-control none -k regex:gemm_kernel -s 1 -c 1 -o /tmp/prof_gemm python bench/ncu_cases.py --case gemm
"""
import argparse
import os
import sys
import threading

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def emulated(world, fn):
    from asystem_amem_b200 import Communicator, get_unique_id
    uid = get_unique_id()
    errs = []

    def body(rank):
        try:
            torch.cuda.set_device(0)
            comm = Communicator(world, rank, uid)
            fn(rank, comm)
            torch.cuda.synchronize()
            comm.destroy()
        except BaseException as e:  # noqa: BLE001
            errs.append(repr(e))

    th = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    if errs:
        raise SystemExit("; ".join(errs))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    reps = args.reps
    if args.case == "gemm":
        from asystem_amem_b200.ops import gemm_bf16
        a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
        b = (torch.randn(3584, 8192, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(8192, 3584, device="cuda", dtype=torch.bfloat16)
        for _ in range(reps):
            gemm_bf16(a, b, out)
        torch.cuda.synchronize()
    elif args.case == "grouped_gemm":
        from asystem_amem_b200.ops import grouped_gemm_bf16, interleave_gate_up
        El, d, ffn, rows = 8, 4096, 1536, 32768
        counts = torch.tensor([5000, 3000, 4097, 4000, 1, 6670, 4000, 6000])
        offs = torch.zeros(El + 1, dtype=torch.int32)
        offs[1:] = counts.cumsum(0)
        offs = offs.cuda()
        x = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
        w13 = interleave_gate_up((torch.randn(El, 2 * ffn, d, device="cuda") * 0.02).to(torch.bfloat16), ffn)
        act = torch.empty(rows, ffn, device="cuda", dtype=torch.bfloat16)
        for _ in range(reps):
            grouped_gemm_bf16(x, w13, offs, out=act, rows_hint=rows, swiglu=True)
        torch.cuda.synchronize()
    elif args.case == "window_allreduce":
        world = 4
        n = 32 << 20  # bf16 elements: 64 MiB per rank

        def fn(rank, comm):
            win = comm.window_alloc(n * 2)
            x = win.tensor(torch.bfloat16, n)
            x.normal_()
            torch.cuda.synchronize()
            for _ in range(reps):
                comm.all_reduce(x, algo="window")
            torch.cuda.synchronize()
            win.free()
        emulated(world, fn)
    elif args.case == "cublas":
        a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
        b = (torch.randn(3584, 8192, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(8192, 3584, device="cuda", dtype=torch.bfloat16)
        for _ in range(reps):
            torch.matmul(a, b.t(), out=out)
        torch.cuda.synchronize()
    elif args.case in ("allreduce", "allgather", "reducescatter", "alltoall", "rs_cast"):
        world = 4
        n = 32 << 20  # bf16 elements per rank: 64 MiB per rank, 256 MiB over the emulated ranks

        def fn(rank, comm):
            x = torch.randn(n, device="cuda").to(torch.bfloat16)
            y = torch.empty(n, device="cuda", dtype=torch.bfloat16)
            for _ in range(reps):
                if args.case == "allreduce":
                    comm.all_reduce(x, y, algo="twoshot")
                elif args.case == "allgather":
                    comm.all_gather(x[: n // world], y)
                elif args.case == "reducescatter":
                    comm.reduce_scatter(x, y[: n // world])
                elif args.case == "rs_cast":
                    comm.reduce_scatter(x.float(), y[: n // world], scale=0.25)
                else:
                    comm.all_to_all(x, y)
        emulated(world, fn)
    elif args.case in ("ag_gemm", "gemm_rs"):
        from asystem_amem_b200.ops import all_gather_gemm, gemm_reduce_scatter
        world = 4

        def fn(rank, comm):
            if args.case == "ag_gemm":
                xs = torch.randn(1024, 8192, device="cuda").to(torch.bfloat16)
                w = (torch.randn(3584, 8192, device="cuda") * 0.02).to(torch.bfloat16)
                for _ in range(reps):
                    all_gather_gemm(comm, xs, w)
            else:
                h = torch.randn(4096, 3584, device="cuda").to(torch.bfloat16)
                w = (torch.randn(8192, 3584, device="cuda") * 0.02).to(torch.bfloat16)
                for _ in range(reps):
                    gemm_reduce_scatter(comm, h, w)
        emulated(world, fn)
    elif args.case == "moe":
        from asystem_amem_b200.ops import MoeDispatcher
        world, T, d, E, k = 4, 8192, 4096, 64, 8

        def fn(rank, comm):
            disp = MoeDispatcher(comm, E, d, 2 * T * k)
            x = torch.randn(T, d, device="cuda").to(torch.bfloat16)
            top = torch.randn(T, E, device="cuda").topk(k, dim=1)
            idx, w = top.indices.to(torch.int32), torch.softmax(top.values, dim=1)
            for _ in range(reps):
                res = disp.dispatch(x, idx)
                disp.combine(idx, w, res.send_pos)
        emulated(world, fn)
    else:
        raise SystemExit(f"unknown case {args.case}")
    print("done", args.case)


if __name__ == "__main__":
    main()
