"""Data parallelism with fully sharded parameters (ZeRO-3 style) on the library's collectives.

Every unit (a decoder block, the embedding, the head) owns one flat bf16 parameter buffer.
Each rank keeps only its 1/n shard (plus an fp32 master copy for the optimizer).  A unit's
forward all-gathers the flat buffer, runs, and frees it; its backward all-gathers again,
recomputes the unit (activation checkpointing at unit granularity), back-propagates, and
reduce-scatters the flat gradient with the averaging scale and the bf16 -> fp32 cast fused into
the reduce-scatter kernel.  The all-gather of the NEXT unit (forward: i + 1, backward: i - 1) is
issued on a side stream before the current unit computes, so it runs under that compute; and the
parameters' ``.grad`` are views into one flat buffer, so the reduce-scatter reads what autograd
wrote, without a packing pass.  All communicator memory is pausable: ``pause_all()`` between steps
gives the staging memory back and ``resume_all()`` restores it without re-initialisation.

Reference parity: none to match -- the reference implements no parallelism strategy, it pauses
whatever communicators a process created (README.md:259, README.md:129-134); this wrapper
exists because the RL co-location use case (README.md:1-60) needs a training step to pause.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn


class _ShardedUnit:
    def __init__(self, module: nn.Module, comm, name: str):
        self.module, self.comm, self.name = module, comm, name
        self.params = [p for p in module.parameters()]
        self.numels = [p.numel() for p in self.params]
        self._shapes = [p.shape for p in self.params]
        total = sum(self.numels)
        n = comm.nranks
        self.padded = int(math.ceil(total / (n * 8)) * n * 8)   # 16-byte aligned shards
        self.shard_len = self.padded // n
        dev = self.params[0].device
        flat = torch.zeros(self.padded, dtype=torch.bfloat16, device=dev)
        off = 0
        for p, k in zip(self.params, self.numels):
            flat[off:off + k] = p.detach().reshape(-1).to(torch.bfloat16)
            off += k
        lo = comm.rank * self.shard_len
        self.shard = flat[lo:lo + self.shard_len].clone()          # bf16 shard that is gathered
        self.master = self.shard.float()                            # fp32 master weights
        self.grad_shard = torch.zeros(self.shard_len, dtype=torch.float32, device=dev)
        for p in self.params:                                       # free the replicated storage
            p.data = torch.empty(0, dtype=p.dtype, device=dev)
        self.full = None
        self._prefetched = None       # (buffer, event) of an all-gather issued ahead of time
        self._gflat = None

    def prefetch(self, side) -> None:
        """Starts this unit's all-gather on ``side`` (CUDA stream); ``gather`` picks it up."""
        if self._prefetched is not None or self.full is not None or side is None:
            return
        with torch.cuda.stream(side):
            buf = torch.empty(self.padded, dtype=torch.bfloat16, device=self.shard.device)
            self.comm.all_gather(self.shard, buf, stream=side)
            ev = torch.cuda.Event()
            ev.record(side)
        self._prefetched = (buf, ev)

    def gather(self) -> None:
        if self._prefetched is not None:
            self.full, ev = self._prefetched
            self._prefetched = None
            torch.cuda.current_stream().wait_event(ev)
            self.full.record_stream(torch.cuda.current_stream())
        else:
            self.full = torch.empty(self.padded, dtype=torch.bfloat16, device=self.shard.device)
            self.comm.all_gather(self.shard, self.full)
        off = 0
        for p, k, shp in zip(self.params, self.numels, self._shapes):
            p.data = self.full[off:off + k].view(shp)
            off += k

    def attach_flat_grads(self) -> None:
        """``.grad`` of every parameter becomes a zeroed view into one flat bf16 buffer: autograd
        accumulates straight into what the reduce-scatter will read."""
        self._gflat = torch.zeros(self.padded, dtype=torch.bfloat16, device=self.shard.device)
        off = 0
        for p, k, shp in zip(self.params, self.numels, self._shapes):
            p.grad = self._gflat[off:off + k].view(shp)
            off += k

    def release(self) -> None:
        dev = self.shard.device
        for p in self.params:
            p.data = torch.empty(0, dtype=p.dtype, device=dev)
        self.full = None

    def reduce_grads(self) -> None:
        flat = self._gflat
        if flat is None:                      # gradients were not attached: pack them
            flat = torch.zeros(self.padded, dtype=torch.bfloat16, device=self.shard.device)
            off = 0
            for p, k in zip(self.params, self.numels):
                if p.grad is not None:
                    flat[off:off + k] = p.grad.reshape(-1)
                off += k
        for p in self.params:
            p.grad = None
        self._gflat = None
        out = torch.empty(self.shard_len, dtype=torch.float32, device=flat.device)
        # sum over ranks, times 1/n, bf16 -> fp32: one kernel
        self.comm.reduce_scatter(flat, out, scale=1.0 / self.comm.nranks)
        self.grad_shard += out


class _UnitFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, unit: _ShardedUnit, anchor, x, *extras):
        # `anchor` requires grad so that the unit joins the graph even when x is an index tensor
        ctx.unit, ctx.extras = unit, extras
        ctx.save_for_backward(x)
        unit.gather()
        if unit.next_unit is not None:
            unit.next_unit.prefetch(unit.side)      # runs under this unit's compute
        with torch.no_grad():
            y = unit.module(x, *extras)
        unit.release()
        return y

    @staticmethod
    def backward(ctx, gy):
        unit = ctx.unit
        (x,) = ctx.saved_tensors
        unit.gather()
        if unit.prev_unit is not None:
            unit.prev_unit.prefetch(unit.side)      # the backward pass visits the units in reverse
        unit.attach_flat_grads()
        with torch.enable_grad():
            xin = x.detach().requires_grad_(x.is_floating_point())
            y = unit.module(xin, *ctx.extras)
            y.backward(gy)
        unit.reduce_grads()
        unit.release()
        return (None, None, xin.grad if x.is_floating_point() else None) + (None,) * len(ctx.extras)


class FSDP:
    """Wraps a model that exposes ``units`` (an iterable of modules called as unit(x, *extras))."""

    def __init__(self, model: nn.Module, comm):
        self.model, self.comm = model, comm
        self.units = [_ShardedUnit(u, comm, f"unit{i}") for i, u in enumerate(model.units)]
        dev = self.units[0].shard.device
        side = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        for i, u in enumerate(self.units):
            u.side = side
            u.next_unit = self.units[i + 1] if i + 1 < len(self.units) else None
            u.prev_unit = self.units[i - 1] if i > 0 else None
        self._anchor = torch.zeros(1, device=self.units[0].shard.device, requires_grad=True)

    def forward_units(self, x, *extras):
        for u in self.units:
            x = _UnitFn.apply(u, self._anchor, x, *extras)
        return x

    def shards(self):
        return [(u.master, u.grad_shard) for u in self.units]

    def zero_grad(self) -> None:
        for u in self.units:
            u.grad_shard.zero_()

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the averaged gradient (all-reduce of the shards' squared sums)."""
        sq = torch.zeros(1, dtype=torch.float32, device=self.units[0].shard.device)
        for u in self.units:
            sq += u.grad_shard.pow(2).sum()
        self.comm.all_reduce(sq)
        return sq.sqrt()

    def sync_shards_from_master(self) -> None:
        for u in self.units:
            u.shard.copy_(u.master)


class ShardedAdamW:
    """AdamW on the fp32 master shards; the bf16 shards that get all-gathered are refreshed after
    every step."""

    def __init__(self, fsdp: FSDP, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0):
        self.fsdp, self.lr, self.betas, self.eps, self.wd = fsdp, lr, betas, eps, weight_decay
        self.m = [torch.zeros_like(u.master) for u in fsdp.units]
        self.v = [torch.zeros_like(u.master) for u in fsdp.units]
        self.t = 0

    @torch.no_grad()
    def step(self) -> None:
        self.t += 1
        b1, b2 = self.betas
        c1, c2 = 1 - b1 ** self.t, 1 - b2 ** self.t
        for u, m, v in zip(self.fsdp.units, self.m, self.v):
            g = u.grad_shard
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            if self.wd:
                u.master.mul_(1 - self.lr * self.wd)
            u.master.addcdiv_(m / c1, (v / c2).sqrt_().add_(self.eps), value=-self.lr)
        self.fsdp.sync_shards_from_master()
