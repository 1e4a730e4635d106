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


    def run_1f1b(self, stage_fn, micro_batches, act_like: torch.Tensor, loss_fn=None):
        """One-forward-one-backward training schedule (PipeDream-flush / Megatron's non-interleaved
        1F1B).  Stage s runs ``n - 1 - s`` warm-up forwards, then alternates one forward with one
        backward, then drains its remaining backwards; at most ``n - s`` micro-batches are alive
        on a stage at any time (GPipe keeps all of them).

        ``stage_fn(x)`` is this stage's differentiable forward; parameter gradients accumulate in
        ``.grad`` over the micro-batches.  ``micro_batches``: on stage 0 the inputs, elsewhere
        only its length matters.  ``loss_fn(y, i)`` (last stage) returns the scalar loss of
        micro-batch ``i``.  Returns the list of losses on the last stage, None elsewhere.
        Every transfer is a send or receive of ``act_like``'s shape and dtype with the
        neighbouring stage, issued in the same order on both sides."""
        m = len(micro_batches)
        first, last = self.stage == 0, self.stage == self.n - 1
        warm = min(self.n - 1 - self.stage, m)
        live = []          # (input that needs a gradient or None, output) of forwards awaiting their backward
        losses = []
        done_f = done_b = 0

        def forward():
            nonlocal done_f
            i = done_f
            done_f += 1
            x = micro_batches[i] if first else self.recv_forward(act_like)
            xin = x if first else x.detach().requires_grad_(True)
            y = stage_fn(xin)
            if last:
                loss = loss_fn(y, i)
                losses.append(loss.detach())
                live.append((xin, loss))
            else:
                self.send_forward(y.detach())
                live.append((xin, y))

        def backward():
            nonlocal done_b
            done_b += 1
            xin, y = live.pop(0)
            if last:
                y.backward()
            else:
                g = self.recv_backward(act_like)
                y.backward(g)
            if not first:
                self.send_backward(xin.grad)

        for _ in range(warm):
            forward()
        for _ in range(m - warm):
            forward()
            backward()
        while done_b < m:
            backward()
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        return losses if last else None


def _is_cpu_comm(comm) -> bool:
    from ..comm import backend_usage
    return backend_usage()["backend"] != "cuda"
