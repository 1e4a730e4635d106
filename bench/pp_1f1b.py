#!/usr/bin/env python
"""Pipeline-parallel 1F1B training step: this library's pausable send / recv against
torch.distributed NCCL point-to-point (the declared baseline) on the same schedule.

One process per GPU, stage s on rank s.  Every stage holds `--layers` residual MLP blocks
(d -> 4d -> d, bf16); a step pushes `--micro` micro-batches of [tokens, d] activations through
the one-forward-one-backward schedule (forward and backward transfers of tokens * d * 2 bytes
between neighbouring stages) and ends with an SGD update.  The communicator is paused and
resumed between the steps of the library arm, as co-located training would do.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29560 bench/pp_1f1b.py

Times are CUDA events on the compute stream around the whole step, max over ranks.

Reference parity: none to match -- the reference has no pipeline code; its send / recv are
NCCL's own (guarded in nccl_patch/nccl_2.27.5-1.diff:113-230).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator  # noqa: E402
from asystem_amem_b200.parallel import PipelineStage  # noqa: E402


class Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.up = nn.Linear(d, 4 * d, bias=False)
        self.down = nn.Linear(4 * d, d, bias=False)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm(x))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--micro", type=int, default=0, help="micro-batches per step (default: 2 x stages)")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="bench_results/pp_1f1b.jsonl")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    dist.all_reduce(torch.zeros(1, device="cuda"))
    gloo = dist.new_group(backend="gloo")
    comm = Communicator.from_torch_distributed(gloo)
    m = args.micro or 2 * world
    torch.manual_seed(rank)
    stage = nn.Sequential(*[Block(args.dim) for _ in range(args.layers)]).cuda().bfloat16()
    opt = torch.optim.SGD(stage.parameters(), lr=1e-4)
    act_like = torch.empty(args.tokens, args.dim, device="cuda", dtype=torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(7)
    inputs = [torch.randn(args.tokens, args.dim, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(m)]

    def loss_fn(y, i):
        return y.float().pow(2).mean()

    def one_step(pipe):
        opt.zero_grad(set_to_none=True)
        losses = pipe.run_1f1b(stage, inputs, act_like, loss_fn)
        opt.step()
        return losses

    def timed(pipe, pause):
        times = []
        last = None
        for it in range(args.warmup + args.steps):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            losses = one_step(pipe)
            e1.record()
            torch.cuda.synchronize()
            if losses:
                last = float(torch.stack(losses).mean())
            if it >= args.warmup:
                t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                times.append(float(t))
            if pause:
                comm.pause()
                comm.resume()
        times.sort()
        return times[len(times) // 2], last

    lib_ms, lib_loss = timed(PipelineStage(comm, rank, world), pause=True)
    nccl_ms, nccl_loss = timed(PipelineStage(comm, rank, world, use_torch_nccl=True), pause=False)
    loss = torch.tensor([lib_loss or 0.0, nccl_loss or 0.0], device="cuda")
    dist.all_reduce(loss, op=dist.ReduceOp.MAX)
    if rank == 0:
        row = {"bench": "pp_1f1b", "n_gpus": world, "stages": world, "micro_batches": m, "tokens": args.tokens, "dim": args.dim,
               "layers_per_stage": args.layers, "bytes_per_transfer": args.tokens * args.dim * 2,
               "amem_step_ms": round(lib_ms, 3), "torch_nccl_p2p_step_ms": round(nccl_ms, 3), "speedup": round(nccl_ms / lib_ms, 3),
               "last_stage_loss_amem": round(float(loss[0]), 5), "last_stage_loss_nccl": round(float(loss[1]), 5),
               "device_errors": comm.async_error()}
        print(json.dumps(row), flush=True)
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "a") as f:
            f.write(json.dumps(row) + "\n")
    dist.barrier()
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
