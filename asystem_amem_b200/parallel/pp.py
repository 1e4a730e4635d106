"""Pipeline parallelism: activations travel between stages with point-to-point transfers.

Two transports: the library's own pausable ncclSend / ncclRecv (default), and
``torch.distributed`` NCCL point-to-point as the declared baseline path (its memory is outside
the registry and is reported separately).  Transfers are issued on a side stream so the next
micro-batch's compute overlaps them; where a stage both sends and receives with the same
neighbour it does so in one grouped exchange (see :func:`plan_1f1b`).

Reference parity: none to match -- the reference has no pipeline code; send/recv are NCCL's
(entry points guarded in nccl_patch/nccl_2.27.5-1.diff:113-230).
"""
from __future__ import annotations

import torch


def plan_1f1b(stage: int, n_stages: int, m: int) -> list:
    """The one-forward-one-backward schedule of one stage as a list of steps.

    Steps: ``("recv_f", i)``, ``("fwd", i)``, ``("send_f", i)``, ``("send_f_recv_b", i, j)``,
    ``("bwd", j)``, ``("send_b", j)``, ``("send_b_recv_f", j, i)``, ``("recv_b", j)`` with
    micro-batch indices i (forward) and j (backward).  Transfers are rendez-vous operations: a
    send completes only while the neighbour runs the matching receive.  In the steady state a stage
    therefore hands its activation forward and takes the next gradient in ONE grouped exchange
    with the next stage (``send_f_recv_b``), and hands its input gradient back and takes the next
    activation in one grouped exchange with the previous stage (``send_b_recv_f``); issued one
    after the other, neighbouring stages would each sit in a send that the other has not reached.
    Steps that do not apply to the first / last stage (no previous / next stage) are left out."""
    first, last = stage == 0, stage == n_stages - 1
    warm = min(n_stages - 1 - stage, m)
    steady = m - warm
    steps = []
    f = b = 0
    for _ in range(warm):
        if not first:
            steps.append(("recv_f", f))
        steps.append(("fwd", f))
        if not last:
            steps.append(("send_f", f))
        f += 1
    if steady and not first:
        steps.append(("recv_f", f))
    for k in range(steady):
        steps.append(("fwd", f))
        if not last:
            steps.append(("send_f_recv_b", f, b))
        f += 1
        steps.append(("bwd", b))
        if not first:
            if k == steady - 1:
                steps.append(("send_b", b))
            else:
                steps.append(("send_b_recv_f", b, f))
        b += 1
    for _ in range(warm):
        if not last:
            steps.append(("recv_b", b))
        steps.append(("bwd", b))
        if not first:
            steps.append(("send_b", b))
        b += 1
    return steps


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

    def _exchange(self, send: torch.Tensor | None, send_peer: int, recv_like: torch.Tensor | None, recv_peer: int):
        """One point-to-point step: a send, a receive, or both as ONE group (both directions then
        run together and neither side waits for the other to finish something else first)."""
        buf = torch.empty_like(recv_like) if recv_like is not None else None
        if send is None and buf is None:
            return None
        if self.use_torch:
            import torch.distributed as dist
            ops = []
            if send is not None:
                ops.append(dist.P2POp(dist.isend, send, send_peer, self.group))
            if buf is not None:
                ops.append(dist.P2POp(dist.irecv, buf, recv_peer, self.group))
            for w in dist.batch_isend_irecv(ops):
                w.wait()
            return buf

        def issue(stream):
            from ..comm import group_end, group_start
            both = send is not None and buf is not None
            if both:
                group_start()
            try:
                if send is not None:
                    self.comm.send(send, send_peer, stream=stream)
                if buf is not None:
                    self.comm.recv(buf, recv_peer, stream=stream)
            finally:
                if both:
                    group_end()

        if self.side is None:
            issue(None)
            return buf
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):
            issue(self.side)
        for t in (send, buf):
            if t is not None:
                t.record_stream(self.side)
        if buf is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        return buf

    def send_forward(self, act: torch.Tensor) -> None:
        if self.stage < self.n - 1:
            self._exchange(act, self.stage + 1, None, -1)

    def recv_forward(self, like: torch.Tensor) -> torch.Tensor | None:
        return None if self.stage == 0 else self._exchange(None, -1, like, self.stage - 1)

    def send_backward(self, grad: torch.Tensor) -> None:
        if self.stage > 0:
            self._exchange(grad, self.stage - 1, None, -1)

    def recv_backward(self, like: torch.Tensor) -> torch.Tensor | None:
        return None if self.stage == self.n - 1 else self._exchange(None, -1, like, self.stage + 1)

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
        1F1B), see :func:`plan_1f1b`.  Stage s runs ``n - 1 - s`` warm-up forwards, then alternates
        one forward with one backward, then drains its remaining backwards; at most ``n - s``
        micro-batches are alive on a stage at any time (GPipe keeps all of them).

        ``stage_fn(x)`` is this stage's differentiable forward; parameter gradients accumulate in
        ``.grad`` over the micro-batches.  ``micro_batches``: on stage 0 the inputs, elsewhere
        only its length matters.  ``loss_fn(y, i)`` (last stage) returns the scalar loss of
        micro-batch ``i``.  Returns the list of losses on the last stage, None elsewhere.
        Every transfer carries ``act_like``'s shape and dtype between neighbouring stages."""
        m = len(micro_batches)
        first, last = self.stage == 0, self.stage == self.n - 1
        prev, nxt = self.stage - 1, self.stage + 1
        live = {}          # micro-batch -> (input that needs a gradient or None, output or loss)
        arrived_f, arrived_b, grads_in = {}, {}, {}
        losses = []
        for step in plan_1f1b(self.stage, self.n, m):
            kind = step[0]
            if kind == "recv_f":
                arrived_f[step[1]] = self._exchange(None, -1, act_like, prev)
            elif kind == "fwd":
                i = step[1]
                x = micro_batches[i] if first else arrived_f.pop(i)
                xin = x if first else x.detach().requires_grad_(True)
                y = stage_fn(xin)
                if last:
                    y = loss_fn(y, i)
                    losses.append(y.detach())
                live[i] = (xin, y)
            elif kind == "send_f":
                self._exchange(live[step[1]][1].detach(), nxt, None, -1)
            elif kind == "send_f_recv_b":
                arrived_b[step[2]] = self._exchange(live[step[1]][1].detach(), nxt, act_like, nxt)
            elif kind == "recv_b":
                arrived_b[step[1]] = self._exchange(None, -1, act_like, nxt)
            elif kind == "bwd":
                j = step[1]
                xin, y = live.pop(j)
                if last:
                    y.backward()
                else:
                    y.backward(arrived_b.pop(j))
                if not first:
                    grads_in[j] = xin.grad
            elif kind == "send_b":
                self._exchange(grads_in.pop(step[1]), prev, None, -1)
            elif kind == "send_b_recv_f":
                arrived_f[step[2]] = self._exchange(grads_in.pop(step[1]), prev, act_like, prev)
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        return losses if last else None


def _is_cpu_comm(comm) -> bool:
    from ..comm import backend_usage
    return backend_usage()["backend"] != "cuda"
