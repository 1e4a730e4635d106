#!/usr/bin/env python
"""Two engines sharing the same GPUs, taking turns: the reference's use case in thirty lines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29560 examples/train_infer_switch.py          # N GPUs
    AMEM_BACKEND=mock python examples/train_infer_switch.py --cpu    # one process, host memory

A "training" communicator (group id 1) and an "inference" communicator (group id 2) live in the
same processes.  While one works the other is paused: its communication buffers are unmapped and
returned to the driver, the communicator object, its peers and its addresses stay valid, and
resuming needs no re-initialisation.  The reference documents the same pattern for SGLang / vLLM
through a ctypes loader (README.md:262-294) and quotes "offload + reload < 1 s per step"
(README.md, RL section); bench/rl_cycle.py is the measured version of this script with a real
model on both sides.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator, get_unique_id, mem_stats  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true", help="single process on the mock backend (no GPU)")
    ap.add_argument("--cycles", type=int, default=3)
    args = ap.parse_args()
    if args.cpu:
        rank, world, device = 0, 1, "cpu"
        train = Communicator(1, 0, get_unique_id())
        infer = Communicator(1, 0, get_unique_id())
    else:
        import torch.distributed as dist
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        device = "cuda"
        dist.init_process_group("gloo", rank=rank, world_size=world)
        train = Communicator.from_torch_distributed()
        infer = Communicator.from_torch_distributed()
    grads = torch.ones(1 << 20, device=device) * (rank + 1)
    acts = torch.ones(1 << 18, device=device)
    infer.pause()                                            # inference starts parked
    for cycle in range(args.cycles):
        train.all_reduce(grads.clone())                      # "training step"
        t0 = time.perf_counter()
        train.pause()                                        # training gives its buffers back ...
        infer.resume()                                       # ... inference takes the GPUs
        switch_ms = (time.perf_counter() - t0) * 1e3
        out = acts.clone()
        infer.all_reduce(out)                                # "decode batch"
        assert float(out[0]) == world
        infer.pause()
        train.resume()
        if rank == 0:
            st = mem_stats()
            print(f"cycle {cycle}: train->infer switch {switch_ms:.2f} ms, "
                  f"live {st['live_bytes'] >> 20} MiB, released by pause {st['paused_bytes'] >> 20} MiB", flush=True)
    infer.resume()
    train.destroy()
    infer.destroy()
    if rank == 0:
        print("switch example ok")


if __name__ == "__main__":
    main()
