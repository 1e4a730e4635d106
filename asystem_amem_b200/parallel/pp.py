"""Pipeline parallelism: activations travel between stages with point-to-point transfers.

Two transports: the library's own pausable ncclSend / ncclRecv (default), and
``torch.distributed`` NCCL point-to-point as the declared baseline path (its memory is outside
the registry and is reported separately).  Transfers are issued on a side stream so the next
micro-batch's compute overlaps them.

Reference parity: none to match -- the reference has no pipeline code; send/recv are NCCL's
(entry points guarded in nccl_patch/nccl_2.27.5-1.diff:113-230).
"""
from __future__ import annotations

import torch


class PipelineStage:
    def __init__(self, comm, stage: int, n_stages: int, use_torch_nccl: bool = False, group=None):
        self.comm, self.stage, self.n = comm, stage, n_stages
        self.use_torch, self.group = use_torch_nccl, group
        self.side = torch.cuda.Stream() if torch.cuda.is_available() and not _is_cpu_comm(comm) else None

    def _on_side(self, fn, tensor):
        if self.side is None:
            return fn(None)
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):
            out = fn(self.side)
        tensor.record_stream(self.side)
        return out

    def send_forward(self, act: torch.Tensor) -> None:
        if self.stage == self.n - 1:
            return
        if self.use_torch:
            import torch.distributed as dist
            dist.send(act, self.stage + 1, group=self.group)
        else:
            self._on_side(lambda s: self.comm.send(act, self.stage + 1, stream=s), act)

    def recv_forward(self, like: torch.Tensor) -> torch.Tensor | None:
        if self.stage == 0:
            return None
        buf = torch.empty_like(like)
        if self.use_torch:
            import torch.distributed as dist
            dist.recv(buf, self.stage - 1, group=self.group)
        else:
            self._on_side(lambda s: self.comm.recv(buf, self.stage - 1, stream=s), buf)
            if self.side is not None:
                torch.cuda.current_stream().wait_stream(self.side)
        return buf

    def send_backward(self, grad: torch.Tensor) -> None:
        if self.stage == 0:
            return
        if self.use_torch:
            import torch.distributed as dist
            dist.send(grad, self.stage - 1, group=self.group)
        else:
            self._on_side(lambda s: self.comm.send(grad, self.stage - 1, stream=s), grad)

    def recv_backward(self, like: torch.Tensor) -> torch.Tensor | None:
        if self.stage == self.n - 1:
            return None
        buf = torch.empty_like(like)
        if self.use_torch:
            import torch.distributed as dist
            dist.recv(buf, self.stage + 1, group=self.group)
        else:
            self._on_side(lambda s: self.comm.recv(buf, self.stage + 1, stream=s), buf)
            if self.side is not None:
                torch.cuda.current_stream().wait_stream(self.side)
        return buf

    def run_gpipe(self, stage_fn, micro_batches, act_like: torch.Tensor):
        """Forward-only GPipe schedule (serving / evaluation): every micro-batch flows through
        the stages; returns the last stage's outputs (None elsewhere)."""
        outs = []
        for mb in micro_batches:
            x = mb if self.stage == 0 else self.recv_forward(act_like)
            y = stage_fn(x)
            if self.stage == self.n - 1:
                outs.append(y)
            else:
                self.send_forward(y)
        return outs if self.stage == self.n - 1 else None


def _is_cpu_comm(comm) -> bool:
    from ..comm import backend_usage
    return backend_usage()["backend"] != "cuda"
