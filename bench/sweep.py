#!/usr/bin/env python
"""Collective bus-bandwidth sweep against stock NCCL (the torch-bundled one), one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29520 bench/sweep.py [--max-bytes 8589934592] [--colls allreduce,allgather,...]

Collectives: allreduce, allgather, reducescatter, alltoall, broadcast, reduce (the reference's run.sh:22 set plus
reduce-scatter).  For every collective, dtype (bf16, fp32) and message size (8 B doubling up to --max-bytes) it
times this library and NCCL with CUDA events on the launching stream (3 warm-ups, L2 flushed
between iterations, max over ranks) and, like the reference's patched nccl-tests, calls
ncclPause()/ncclResume() once between sizes.  busBW follows nccl-tests: all-reduce
algBW*2(n-1)/n; all-gather, reduce-scatter, all-to-all algBW*(n-1)/n.

Reference parity: the reference's own test is this sweep on nccl-tests binaries (run.sh:22-30:
all_reduce_perf, all_gather_perf, alltoall_perf, broadcast_perf, -b 4M -e 8M -f 2) with one
ncclPause / ncclResume after every size (nccl_patch/nccl-tests.diff:24-50).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator, pause_all, resume_all  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--factor", type=int, default=2)
    ap.add_argument("--colls", default="allreduce,allgather,reducescatter,alltoall")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--no-pause", action="store_true")
    ap.add_argument("--window", action="store_true",
                    help="all-reduce between two registered windows (ncclMemAlloc + ncclCommWindowRegister): in place on the peers' "
                         "memory, no staging; NCCL gets buffers from its own registered memory pool as the like-for-like arm")
    ap.add_argument("--out", default="bench_results/sweep.jsonl")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    dist.all_reduce(torch.zeros(1, device="cuda"))
    gloo = dist.new_group(backend="gloo")
    comm = Communicator.from_torch_distributed(gloo)
    info = comm.info()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    out_f = open(args.out, "a") if rank == 0 else None
    dts = {"bf16": torch.bfloat16, "fp32": torch.float32}
    win_a = win_b = None
    nccl_pool = None
    if args.window:
        win_a, win_b = comm.window_alloc(args.max_bytes), comm.window_alloc(args.max_bytes)
        try:   # NCCL's user-buffer registration: tensors from a pool backed by ncclMemAlloc, registered with the communicator
            backend = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda"))
            nccl_pool = torch.cuda.MemPool(backend.mem_allocator)
            with torch.cuda.use_mem_pool(nccl_pool):
                nccl_buf = torch.empty(args.max_bytes, dtype=torch.uint8, device="cuda")
            backend.register_mem_pool(nccl_pool)
        except Exception as e:  # noqa: BLE001
            nccl_pool = None
            if rank == 0:
                print(json.dumps({"nccl_registered_pool": f"unavailable: {type(e).__name__}: {e}"}), flush=True)

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier(group=gloo)
        total = 0.0
        for _ in range(iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        t = torch.tensor([total / iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return float(t.item())

    for coll in args.colls.split(","):
        for dn in args.dtypes.split(","):
            dt = dts[dn]
            es = torch.empty(0, dtype=dt).element_size()
            size = args.min_bytes
            while size <= args.max_bytes:
                n = max(1, size // es)
                if coll != "allreduce":
                    n = max(world, n // world * world)
                nbytes = n * es
                iters = 20 if nbytes <= (64 << 20) else 5
                x = torch.randn(n, device="cuda", dtype=torch.float32).to(dt)
                y = torch.empty_like(x)
                ref_reg = None
                if coll == "allreduce":
                    if args.window:
                        xw, yw = win_a.tensor(dt, n), win_b.tensor(dt, n)
                        xw.copy_(x)
                        ours = lambda: comm.all_reduce(xw, yw)
                        if nccl_pool is not None:
                            yr = nccl_buf[:nbytes].view(dt)
                            ref_reg = lambda: dist.all_reduce(yr)
                    else:
                        ours = lambda: comm.all_reduce(x, y)
                    ref = lambda: dist.all_reduce(y)
                    factor = 2 * (world - 1) / world
                elif coll == "broadcast":
                    ours = lambda: comm.broadcast(x, y, root=0)
                    ref = lambda: dist.broadcast(y, src=0)
                    factor = 1.0
                elif coll == "reduce":
                    ours = lambda: comm.reduce(x, y, root=0)
                    ref = lambda: dist.reduce(y, dst=0)
                    factor = 1.0
                elif coll == "allgather":
                    ours = lambda: comm.all_gather(x[: n // world], y)
                    ref = lambda: dist.all_gather_into_tensor(y, x[: n // world])
                    factor = (world - 1) / world
                elif coll == "reducescatter":
                    ours = lambda: comm.reduce_scatter(x, y[: n // world])
                    ref = lambda: dist.reduce_scatter_tensor(y[: n // world], x)
                    factor = (world - 1) / world
                else:
                    ours = lambda: comm.all_to_all(x, y)
                    ref = lambda: dist.all_to_all_single(y, x)
                    factor = (world - 1) / world
                t_ours = timed(ours, iters)
                t_ref = timed(ref, iters)
                row = {"coll": coll, "dtype": dn, "bytes": nbytes, "n_gpus": world, "nvls": info["nvls"],
                       "amem_us": round(t_ours * 1e3, 2), "nccl_us": round(t_ref * 1e3, 2),
                       "amem_busbw_gbs": round(nbytes / (t_ours * 1e-3) * factor / 1e9, 2),
                       "nccl_busbw_gbs": round(nbytes / (t_ref * 1e-3) * factor / 1e9, 2),
                       "speedup": round(t_ref / t_ours, 3)}
                if args.window and coll == "allreduce":
                    row["window"] = True
                    if ref_reg is not None:
                        t_reg = timed(ref_reg, iters)
                        row["nccl_registered_us"] = round(t_reg * 1e3, 2)
                        row["nccl_registered_busbw_gbs"] = round(nbytes / (t_reg * 1e-3) * factor / 1e9, 2)
                if not args.no_pause:
                    pause_all()
                    resume_all()
                    st = comm.pause_resume_stats()
                    row["pause_ms"] = round(st["pause_total_us"] / 1e3, 3)
                    row["resume_ms"] = round(st["resume_total_us"] / 1e3, 3)
                if rank == 0:
                    line = json.dumps(row)
                    print(line, flush=True)
                    out_f.write(line + "\n")
                    out_f.flush()
                del x, y
                size *= args.factor
    err = comm.async_error()
    if rank == 0:
        print(json.dumps({"device_errors": err}), flush=True)
    if win_a is not None:
        win_b.free()
        win_a.free()
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
