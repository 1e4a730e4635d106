#!/usr/bin/env python
"""Headline benchmark: the reference's own test cycle at the reference's own footprint.

The reference's harness (its nccl-tests patch, nccl_patch/nccl-tests.diff:24-50) runs a collective,
calls ncclPause(), then ncclResume(), and runs the collective again without re-initialising
anything; its published 8-GPU run released 3076 MB per GPU (docs/images/run_result.webp).  One
bench step does exactly that — all-reduce -> pause -> resume -> all-reduce — on N GPUs of one node
(one process per GPU, launched by torch.distributed.run for N > 1), with a communicator that holds
``--stage-mb`` of buffers shared with every peer plus ``--stateful-mb`` of user memory whose
contents must survive (an ncclMemAlloc buffer), 3264 MiB per GPU by default.

Three arms, same step, same footprint, same statistics:
  --impl amem        this library (default)
  --impl reference   the unmodified reference plugin (baseline/_ref/lib/libamem_nccl.so.1) driven
                     through its own entry points the way its NCCL patch drives it
                     (baseline/ref_harness.cc, baseline/ref_arm.py).  Its collectives are stock NCCL
                     (the reference ships no kernels of its own: its collectives ARE NCCL's), so the
                     all-reduce of this arm is torch.distributed's NCCL.
  --impl nccl-reinit stock NCCL, "pause" = destroy the communicator, "resume" = create it again

Reported (one JSON line from rank 0):
  value              pause + resume latency in ms: per step the max over ranks, then the median
                     over the timed steps (p90 and mean alongside)
  gib_freed_per_gpu  device memory returned to the driver by the pause (cudaMemGetInfo delta)
  busbw_gbs          bus bandwidth of the all-reduce inside the step (CUDA events, max over ranks)
  e2e                the whole cycle through the public API including the host->device copy of the
                     step's input from pinned memory and the device->host read of the result
  verified           contents of the stateful memory after every resume, and (N >= 2) the
                     post-resume all-reduce against an fp32 sum computed on the CPU ranks
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PUBLISHED_MS = 1000.0  # the reference's published steady-state figure: "< 1 second" per offload+reload (README.md:17,25)


class RawCudaBuffer:
    """Lets torch view device memory that a C library allocated (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes // 4,), "typestr": "<i4", "data": (ptr, False), "version": 2}


def percentile(v, q):
    s = sorted(v)
    return s[min(len(s) - 1, int(round(q * (len(s) - 1))))]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="amem", choices=["amem", "reference", "nccl-reinit"])
    ap.add_argument("--mib", type=int, default=256, help="all-reduce message size in MiB (bf16); larger than the 126 MB L2")
    ap.add_argument("--stage-mb", type=int, default=3072, help="communicator buffers shared with every peer, MiB per GPU")
    ap.add_argument("--stateful-mb", type=int, default=192, help="user memory (ncclMemAlloc) saved and restored across the pause, MiB per GPU")
    ap.add_argument("--records", type=int, default=1, help="number of shared allocations the --stage-mb bytes are spread over")
    ap.add_argument("--ref-limit-s", type=int, default=900, help="wall-clock limit of the reference arm (its host waits are unbounded)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    args.gpus = world
    multi = world > 1
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    real_stdout = None

    def emit(obj: dict) -> None:
        line = json.dumps(obj) + "\n"
        if real_stdout is not None:
            os.write(real_stdout, line.encode())
        else:
            sys.stdout.write(line)
            sys.stdout.flush()

    if args.impl == "reference":
        from baseline import ref_arm
        ok, why = ref_arm.available()
        if not ok:
            if rank == 0:
                emit({"impl": "reference", "unavailable": why})
            return
        ref_arm.restrict_visible_devices(world)       # before CUDA comes up in this process
        # the plugin logs with printf on stdout; the JSON line must stay alone there
        sys.stdout.flush()
        real_stdout = os.dup(1)
        log = os.open(os.path.join(os.environ.get("AMEM_REF_LOG_DIR", "/tmp"), f"amem_ref_arm_rank{rank}.log"), os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
        os.dup2(log, 1)

        def expired():
            if rank == 0:
                emit({"impl": "reference", "unavailable": f"the reference did not finish within {args.ref_limit_s} s (its host-side waits have no deadline)"})
            os._exit(0)
        watchdog = threading.Timer(args.ref_limit_s, expired)
        watchdog.daemon = True
        watchdog.start()

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    gloo = None
    if multi:
        if args.impl == "amem":
            dist.init_process_group("gloo", rank=rank, world_size=world)
            gloo = dist.group.WORLD
        else:
            dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
            # (the re-init arm destroys and re-creates the default group every step: it uses that one throughout)
            gloo = dist.new_group(backend="gloo") if args.impl == "reference" else None

    def host_barrier():
        if multi:
            dist.barrier(group=gloo)

    def max_over_ranks_vec(v):
        t = torch.tensor(v, dtype=torch.float64)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return t.tolist()

    def sum_over_ranks(v: int) -> int:
        t = torch.tensor([v], dtype=torch.int64)
        if multi:
            dist.all_reduce(t, group=gloo)
        return int(t.item())

    n_elem = args.mib * (1 << 20) // 2
    host_in = torch.randn(n_elem, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    host_out = torch.empty(16, dtype=torch.float32).pin_memory()
    x = torch.empty(n_elem, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    stage_bytes, stateful_bytes = args.stage_mb << 20, args.stateful_mb << 20
    launches_per_step = 0
    footprint = {}

    # ---- the three arms: collective / pause / resume / touch / verify ------------------------------
    if args.impl == "amem":
        # one shared allocation: the staging segment itself; several: 288 MiB of staging, the rest as windows
        os.environ["AMEM_STAGE_MB"] = str(args.stage_mb if args.records <= 1 else min(288, args.stage_mb))
        from asystem_amem_b200 import Communicator, get_unique_id, mem_stats, pause_all, process_pause_resume_stats, resume_all
        from asystem_amem_b200.comm import backend_timings, mem_alloc
        comm = Communicator.from_torch_distributed() if multi else Communicator(1, 0, get_unique_id())
        windows = []
        if args.records > 1:   # the shared bytes as registered windows: each one imported by every peer
            each = max(2 << 20, (stage_bytes - (288 << 20)) // args.records)
            for _ in range(args.records):
                windows.append(comm.window_alloc(each))
        user = None
        if stateful_bytes:
            user_ptr = mem_alloc(stateful_bytes)
            user = torch.as_tensor(RawCudaBuffer(user_ptr, stateful_bytes), device="cuda")
        launches_per_step = 2   # two all-reduce kernels of this library per step; pause / resume launch none

        def collective():
            comm.all_reduce(x, y)

        def pause():
            pause_all()

        def resume():
            resume_all()

        def touch(step):
            if user is not None:
                user.fill_(0x5A000000 + step)

        def verify(step) -> int:
            if user is None:
                return 0
            return int((user != 0x5A000000 + step).sum().item())

        def mem_free():
            return torch.cuda.mem_get_info()[0]
    elif args.impl == "reference":
        arm = ref_arm.ReferenceArm(rank, world, local, stage_bytes, args.records, stateful_bytes, host_barrier)
        footprint = arm.tracked_bytes()

        def collective():
            dist.all_reduce(y.copy_(x)) if multi else y.copy_(x)

        pause, resume, touch, verify, mem_free = arm.pause, arm.resume, arm.touch, arm.verify, arm.mem_free
    else:
        def collective():
            dist.all_reduce(y.copy_(x)) if multi else y.copy_(x)

        def pause():  # stock NCCL can only give memory back by destroying the communicator
            if multi:
                torch.cuda.synchronize()
                dist.destroy_process_group()

        def resume():
            if multi:
                dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
                dist.all_reduce(torch.zeros(1, device="cuda"))

        def touch(step):
            pass

        def verify(step) -> int:
            return 0

        def mem_free():
            return torch.cuda.mem_get_info()[0]

    from asystem_amem_b200.utils.timing import ClockSampler   # in-process NVML, initialised before the timed region
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    bad_words = 0

    def step(i: int, record: bool):
        """One cycle.  Returns (pause_ms, resume_ms, allreduce_ms, freed_bytes, e2e_ms)."""
        nonlocal bad_words
        host_barrier()      # every rank has finished checking the previous step (ranks read each other's memory there)
        touch(i)
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
        free0 = mem_free()
        t1 = time.perf_counter()
        pause()
        t2 = time.perf_counter()
        if args.impl == "reference":
            host_barrier()                                       # the reference leaves this barrier to its caller (README.md:160-171):
        t2a = time.perf_counter()                                # counted in e2e, not in pause / resume
        free1 = mem_free()                                       # instrumentation, outside every timed window (pages of shared
        t2b = time.perf_counter()                                # memory return once every rank has let go: after the barrier)
        resume()
        t3 = time.perf_counter()
        collective()
        host_out.copy_(y[:16].float(), non_blocking=True)        # D2H read of the result
        torch.cuda.synchronize()
        t4 = time.perf_counter()
        ar_ms = ev[0].elapsed_time(ev[1])
        bad_words += verify(i)
        return (t2 - t1) * 1e3, (t3 - t2b) * 1e3, ar_ms, free1 - free0, (t4 - t0 - (t2b - t2a)) * 1e3

    # NVML comes up here, before any timed step; clocks are read once per step while the timed
    # all-reduce runs on the GPU (never across pause / resume, which such queries slow down)
    sampler = ClockSampler(local, period_s=None)
    for i in range(args.warmup):
        step(i, False)
    if args.impl == "amem":
        backend_timings(reset=True)
    bad_words = 0
    rows = []
    torch.cuda.synchronize()
    host_barrier()
    with sampler as clocks:
        t_begin = time.perf_counter()
        for i in range(args.steps):
            rows.append(step(args.warmup + i, True))
        torch.cuda.synchronize()
        host_barrier()
        t_end = time.perf_counter()

    # ---- correctness of the post-resume collective (outside the timed region) ----------------------
    verified = bad_words == 0
    allreduce_checked = False
    if multi and args.impl != "nccl-reinit":
        n_chk = 1 << 20
        x.copy_(host_in, non_blocking=True)
        x.mul_(float(rank + 1) / world)                          # ranks contribute different data
        collective()
        torch.cuda.synchronize()
        ref = x[:n_chk].float().cpu().double()
        dist.all_reduce(ref, group=gloo)
        got = y[:n_chk].float().cpu().double()
        err = (got - ref).abs()
        tol = 2.0 ** -7 * ref.abs() + 2.0 ** -6                  # one bf16 rounding of the sum plus the summands' own
        allreduce_checked = True
        if not bool((err <= tol).all()):
            verified = False
            print(f"rank {rank}: post-resume all-reduce differs from the fp32 sum: max err {float(err.max())}", file=sys.stderr)
    verified = sum_over_ranks(0 if verified else 1) == 0

    per_step = max_over_ranks_vec([r[0] + r[1] for r in rows])
    pause_v = max_over_ranks_vec([r[0] for r in rows])
    resume_v = max_over_ranks_vec([r[1] for r in rows])
    ar_v = max_over_ranks_vec([r[2] for r in rows])
    e2e_v = max_over_ranks_vec([r[4] for r in rows])
    ms_per_step = max_over_ranks_vec([(t_end - t_begin) * 1e3 / args.steps])[0]
    freed = min(r[3] for r in rows)
    nbytes = n_elem * 2
    ar_ms = statistics.median(ar_v)
    busbw = (nbytes / (ar_ms * 1e-3)) * (2 * (world - 1) / world if world > 1 else 1.0) / 1e9
    detail = {}
    if args.impl == "amem":
        detail = {k: round(v, 1) if isinstance(v, float) else v for k, v in process_pause_resume_stats().items()}
        detail["driver_calls_rank0_all_steps"] = backend_timings()
        ms = mem_stats()
        footprint = {"local_records": ms["n_local"], "imported_records": ms["n_imported"], "stateful_bytes": ms["stateful_bytes"],
                     "scratch_bytes": ms["scratch_bytes"], "imported_bytes": ms["imported_bytes"]}
    if rank == 0:
        value = statistics.median(per_step)
        emit({
            "metric": "pause+resume ms (GiB freed/GPU and all-reduce busBW alongside)", "impl": args.impl,
            "value": round(value, 3), "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 3), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": round(value / PUBLISHED_MS, 5), "dtype": "bf16", "data": "synthetic N(0,1), random init",
            "statistic": "median over steps of the per-step max over ranks",
            "p90_ms": round(percentile(per_step, 0.9), 3), "mean_ms": round(statistics.mean(per_step), 3),
            "pause_ms": round(statistics.median(pause_v), 3), "resume_ms": round(statistics.median(resume_v), 3),
            "gib_freed_per_gpu": round(freed / 2**30, 4),
            "allreduce_ms": round(ar_ms, 4), "busbw_gbs": round(busbw, 2),
            "allreduce_impl": "this library's kernels" if args.impl == "amem" else "stock NCCL (torch.distributed)" if multi else "device copy",
            "verified": verified, "allreduce_checked": allreduce_checked,
            "config": {"model": "nccl-tests style cycle: all_reduce -> ncclPause -> ncclResume -> all_reduce",
                       "global_batch": world, "seq_len": n_elem, "message_bytes": nbytes,
                       "stage_mb": args.stage_mb, "stateful_mb": args.stateful_mb, "records": args.records, "footprint": footprint,
                       "parallelism": f"dp{world}", "l2": "inputs larger than L2 (256 MiB message)",
                       "baseline_number": "reference README: offload+reload < 1 s per step (Hopper); its 8-GPU test run released 3076 MB per GPU"},
            "e2e": {"value": round(statistics.median(e2e_v), 3), "unit": "ms per cycle incl. H2D input and D2H result",
                    "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 64},
            "gpu_launches": launches_per_step * args.steps, "clocks": clocks.summary(), "phases_us": detail,
        })
    if args.impl == "reference":
        # the plugin's threads and sockets have no shutdown path: leave without running its destructors
        sys.stdout.flush()
        host_barrier()
        os._exit(0)
    if multi and dist.is_initialized():
        if args.impl == "amem":
            comm.destroy()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
