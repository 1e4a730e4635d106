"""Expert parallelism with gradients, on the fused dispatch / combine kernels.

Forward of one MoE layer on every rank of the expert-parallel communicator::

    rows[pos(t, c)] = x[t]                      dispatch  (permute inside the all-to-all)
    y               = experts(rows)             local, grouped by expert
    out[t]          = sum_c w[t, c] * y[pos(t, c)]   combine (un-permute + weighted sum)

Both communication steps are linear maps whose transposes are each other, so the backward pass
runs on the same two kernels and needs no new device code:

* d out / d y  : ``g_y[pos(t, c)] = w[t, c] * g_out[t]`` is a dispatch of the ``T * k`` scaled
  rows with one choice per row.  The kernels place rows by (expert, source rank, pair order), and
  the flattened pair order of the ``[T * k, 1]`` problem is the pair order of the ``[T, k]`` one,
  so every row lands exactly where its forward row was.
* d out / d w  : ``g_w[t, c] = <g_out[t], y[pos(t, c)]>`` needs the expert outputs back at their
  tokens: a combine of the ``[T * k, 1]`` problem with unit weights is that gather.
* d rows / d x : ``g_x[t] = sum_c g_rows[pos(t, c)]`` is a combine with unit weights.

The four steps are plain functions (``dispatch_forward`` ... ``combine_backward``) so that a
caller which schedules its own backward pass -- or a test that runs several ranks as threads of
one process, where the autograd engine's single per-device thread could not run the ranks'
collectives side by side -- can call them directly; ``ep_dispatch`` / ``ep_combine`` wrap them
as autograd functions for everybody else.  Every rank must run the same sequence of steps.

The reference library stops at the communication layer (its all-to-all is NCCL's grouped
send/recv kept alive across ncclPause/ncclResume); routing, permutation and their gradients are
left to the training framework above it.
"""
from __future__ import annotations

import torch

from ..ops.moe import DispatchResult, MoeDispatcher  # noqa: F401


def dispatch_forward(disp: MoeDispatcher, x: torch.Tensor, idx: torch.Tensor):
    """Returns (rows, expert_offsets, send_pos, total): ``rows`` is a private copy of the
    received rows (the receive buffer is reused by the next dispatch)."""
    res = disp.dispatch(x.contiguous(), idx)
    total = int(res.expert_offsets[-1].item())  # host sync: the group boundaries are needed on the host anyway
    return res.recv_x[:total].clone(), res.expert_offsets, res.send_pos, total


def dispatch_backward(disp: MoeDispatcher, g_rows: torch.Tensor, idx: torch.Tensor, send_pos: torch.Tensor) -> torch.Tensor:
    T, k = idx.shape
    disp.y[: g_rows.shape[0]] = g_rows.to(torch.bfloat16)
    ones = torch.ones(T, k, dtype=torch.float32, device=g_rows.device)
    return disp.combine(idx, ones, send_pos)


def combine_forward(disp: MoeDispatcher, y_rows: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, send_pos: torch.Tensor) -> torch.Tensor:
    disp.y[: y_rows.shape[0]] = y_rows.to(torch.bfloat16)
    return disp.combine(idx, w, send_pos)


def combine_backward(disp: MoeDispatcher, g_out: torch.Tensor, y_rows: torch.Tensor, idx: torch.Tensor, w: torch.Tensor,
                     send_pos: torch.Tensor):
    """Returns (g_y_rows, g_w)."""
    T, k = idx.shape
    d = g_out.shape[1]
    flat_idx = idx.reshape(T * k, 1)
    # expert outputs back at their (token, choice): the gather for the routing-weight gradient
    disp.y[: y_rows.shape[0]] = y_rows.to(torch.bfloat16)
    ones = torch.ones(T * k, 1, dtype=torch.float32, device=g_out.device)
    y_at = disp.combine(flat_idx, ones, send_pos.reshape(T * k))
    g_w = (y_at.view(T, k, d).float() * g_out.float().unsqueeze(1)).sum(-1)
    # scaled output gradients to the experts, landing row for row where the forward rows were
    scaled = (g_out.float().unsqueeze(1) * w.float().unsqueeze(2)).to(torch.bfloat16).view(T * k, d)
    res = disp.dispatch(scaled, flat_idx)
    return res.recv_x[: y_rows.shape[0]].clone(), g_w


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, disp):
        rows, offsets, send_pos, _ = dispatch_forward(disp, x, idx)
        ctx.disp = disp
        ctx.save_for_backward(idx, send_pos)
        ctx.mark_non_differentiable(offsets, send_pos)
        return rows, offsets, send_pos

    @staticmethod
    def backward(ctx, g_rows, _g_off, _g_pos):
        idx, send_pos = ctx.saved_tensors
        return dispatch_backward(ctx.disp, g_rows.contiguous(), idx, send_pos), None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_rows, w, idx, send_pos, disp):
        ctx.disp = disp
        ctx.save_for_backward(y_rows, w, idx, send_pos)
        return combine_forward(disp, y_rows, idx, w, send_pos)

    @staticmethod
    def backward(ctx, g_out):
        y_rows, w, idx, send_pos = ctx.saved_tensors
        g_y, g_w = combine_backward(ctx.disp, g_out.contiguous(), y_rows, idx, w, send_pos)
        return g_y, g_w.to(w.dtype), None, None, None


def ep_dispatch(disp: MoeDispatcher, x: torch.Tensor, idx: torch.Tensor):
    """Differentiable dispatch: (rows grouped by local expert, expert_offsets, send_pos)."""
    return _Dispatch.apply(x, idx.to(torch.int32).contiguous(), disp)


def ep_combine(disp: MoeDispatcher, y_rows: torch.Tensor, w: torch.Tensor, idx: torch.Tensor, send_pos: torch.Tensor) -> torch.Tensor:
    """Differentiable combine of the experts' outputs (rows in dispatch order) with weights ``w``."""
    return _Combine.apply(y_rows, w, idx.to(torch.int32).contiguous(), send_pos, disp)
