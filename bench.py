#!/usr/bin/env python
"""Headline benchmark: the reference's own test cycle, on this library.

The reference's harness (its nccl-tests patch) runs a collective, calls ncclPause(), then
ncclResume(), and runs the collective again without re-initialising anything.  One bench step
does exactly that: all-reduce -> ncclPause(NULL) -> ncclResume(NULL) -> all-reduce, on N GPUs
of one node (one process per GPU, launched by torch.distributed.run for N > 1).

Reported (one JSON line from rank 0):
  value            pause+resume latency in ms, max over ranks, mean over the timed steps
  gib_freed_per_gpu  device memory returned to the driver by ncclPause (cudaMemGetInfo delta)
  busbw_gbs        bus bandwidth of the all-reduce inside the step (CUDA events, max over ranks)
  e2e              the whole cycle through the public Python API including the host->device
                   copy of the step's input from pinned memory and the device->host read of
                   the result
`--impl reference` would run the reference's patched NCCL; it cannot be built offline (its NCCL
and nccl-tests submodules are empty and there is no mpirun), so that arm reports unavailable.
`--impl nccl-reinit` is the stock-NCCL stand-in (destroy + re-create the communicator).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PUBLISHED_MS = 1000.0  # the reference's published steady-state figure: "< 1 second" per offload+reload


from asystem_amem_b200.utils.timing import ClockSampler  # noqa: E402  (in-process NVML, initialised before the timed region)


def reference_arm(args) -> None:
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = ("reference is a patch to NCCL 2.27.5 plus a C++ plugin: no Python package to pip-install, its third_party/nccl "
           "and nccl-tests submodules are empty, there is no network and no mpirun")
    if os.path.isdir(ref) and os.listdir(ref):
        why = "baseline/_ref holds no runnable patched-NCCL build (needs the NCCL 2.27.5 and nccl-tests sources and mpirun)"
    if int(os.environ.get("RANK", "0")) == 0:   # one line per job, also under torchrun
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="amem", choices=["amem", "reference", "nccl-reinit"])
    ap.add_argument("--mib", type=int, default=256, help="all-reduce message size in MiB (bf16); larger than the 126 MB L2")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo" if args.impl == "amem" else "nccl", rank=rank, world_size=world)

    def host_barrier():
        if multi:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if not multi:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda" if args.impl != "amem" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n_elem = args.mib * (1 << 20) // 2
    host_in = torch.randn(n_elem, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    host_out = torch.empty(16, dtype=torch.float32).pin_memory()
    x = torch.empty(n_elem, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    launches = 0

    if args.impl == "amem":
        from asystem_amem_b200 import Communicator, get_unique_id, pause_all, process_pause_resume_stats, resume_all
        from asystem_amem_b200.comm import backend_timings
        comm = Communicator.from_torch_distributed() if multi else Communicator(1, 0, get_unique_id())

        def collective():
            comm.all_reduce(x, y)

        def pause():
            pause_all()

        def resume():
            resume_all()
    else:
        def collective():
            dist.all_reduce(y.copy_(x)) if multi else y.copy_(x)

        def pause():  # stock NCCL can only give memory back by destroying the communicator
            if multi:
                torch.cuda.synchronize()
                dist.destroy_process_group()

        def resume():
            if multi:
                dist.init_process_group("nccl", rank=rank, world_size=world)
                dist.all_reduce(torch.zeros(1, device="cuda"))

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]

    def step(record: bool):
        """One cycle.  Returns (pause_ms, resume_ms, allreduce_ms, freed_bytes, e2e_ms)."""
        torch.cuda.synchronize()
        host_barrier()
        t0 = time.perf_counter()
        x.copy_(host_in, non_blocking=True)                      # H2D of this step's input
        torch.cuda.synchronize()
        host_barrier()                                           # ranks enter the collective together
        ev[0].record()
        collective()
        ev[1].record()
        if record:
            sampler.sample_now()                                 # the kernel is still running: clocks under load
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        t1 = time.perf_counter()
        pause()
        t2 = time.perf_counter()
        free1 = torch.cuda.mem_get_info()[0]                     # instrumentation, outside both timed windows
        t2b = time.perf_counter()
        resume()
        t3 = time.perf_counter()
        collective()
        host_out.copy_(y[:16].float(), non_blocking=True)        # D2H read of the result
        torch.cuda.synchronize()
        t4 = time.perf_counter()
        return (t2 - t1) * 1e3, (t3 - t2b) * 1e3, ev[0].elapsed_time(ev[1]), free1 - free0, (t4 - t0) * 1e3

    # NVML comes up here, before any timed step; clocks are read once per step while the timed
    # all-reduce runs on the GPU (never across ncclPause / ncclResume, which such queries slow down)
    sampler = ClockSampler(local, period_s=None)
    for _ in range(args.warmup):
        step(False)
    if args.impl == "amem":
        backend_timings(reset=True)
    rows = []
    torch.cuda.synchronize()
    host_barrier()
    with sampler as clocks:
        t_begin = time.perf_counter()
        for _ in range(args.steps):
            rows.append(step(True))
            launches += 2
        torch.cuda.synchronize()
        host_barrier()
        t_end = time.perf_counter()
    pause_ms = max_over_ranks(statistics.mean(r[0] for r in rows))
    resume_ms = max_over_ranks(statistics.mean(r[1] for r in rows))
    ar_ms = max_over_ranks(statistics.mean(r[2] for r in rows))
    e2e_ms = max_over_ranks(statistics.mean(r[4] for r in rows))
    freed = min(r[3] for r in rows)
    ms_per_step = max_over_ranks((t_end - t_begin) * 1e3 / args.steps)
    nbytes = n_elem * 2
    busbw = (nbytes / (ar_ms * 1e-3)) * (2 * (world - 1) / world if world > 1 else 1.0) / 1e9
    detail = {}
    if args.impl == "amem":
        detail = {k: round(v, 1) if isinstance(v, float) else v for k, v in process_pause_resume_stats().items()}
        detail["driver_calls_rank0_all_steps"] = backend_timings()
    if rank == 0:
        value = pause_ms + resume_ms
        print(json.dumps({
            "metric": "pause+resume ms (GiB freed/GPU and all-reduce busBW alongside)", "impl": args.impl,
            "value": round(value, 3), "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 3), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": round(value / PUBLISHED_MS, 5), "dtype": "bf16", "data": "synthetic N(0,1), random init",
            "pause_ms": round(pause_ms, 3), "resume_ms": round(resume_ms, 3),
            "gib_freed_per_gpu": round(freed / 2**30, 4),
            "allreduce_ms": round(ar_ms, 4), "busbw_gbs": round(busbw, 2),
            "config": {"model": "nccl-tests style cycle: all_reduce -> ncclPause -> ncclResume -> all_reduce",
                       "global_batch": world, "seq_len": n_elem, "message_bytes": nbytes,
                       "parallelism": f"dp{world}", "l2": "inputs larger than L2 (256 MiB message)",
                       "baseline_number": "reference README: offload+reload < 1 s per step (Hopper)"},
            "e2e": {"value": round(e2e_ms, 3), "unit": "ms per cycle incl. H2D input and D2H result",
                    "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 64},
            "gpu_launches": launches, "clocks": clocks.summary(), "phases_us": detail,
        }), flush=True)
    if multi and dist.is_initialized():
        if args.impl == "amem":
            comm.destroy()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
