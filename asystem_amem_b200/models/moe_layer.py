"""Expert-parallel MoE layer: top-k softmax routing, fused dispatch (permute inside the
all-to-all), the experts' SwiGLU FFN as two grouped tcgen05 GEMMs over all local experts at once
(group boundaries read on the device from the dispatch's ``expert_offsets``), fused combine
(un-permute + weighted sum while pulling the rows back).

Without gradients nothing of a layer's forward returns to the host: dispatch -> grouped GEMM with
the SwiGLU epilogue -> grouped GEMM straight into the combine buffer -> combine.  With gradients
the two communication steps run as autograd functions whose backward passes reuse the same kernels
(parallel/ep.py) and the expert GEMMs are :class:`GroupedLinear` (forward and input gradient on the
grouped kernel; the weight gradient, a GEMM with a ragged inner dimension, is a per-expert matmul
and reads the group boundaries on the host).

Reference parity: none -- the reference keeps NCCL's all-to-all buffers alive across
ncclPause / ncclResume (README.md:132) and leaves the layer to the framework above it."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.gemm import grouped_gemm_bf16, interleave_gate_up
from ..ops.moe import MoeDispatcher
from ..parallel.ep import ep_combine, ep_dispatch


class GroupedLinear(torch.autograd.Function):
    """out[rows of group e] = rows @ w[e].T for every group, differentiable."""

    @staticmethod
    def forward(ctx, rows, w, offsets):
        ctx.save_for_backward(rows, w, offsets)
        return grouped_gemm_bf16(rows.contiguous(), w.contiguous(), offsets, rows_hint=rows.shape[0])

    @staticmethod
    def backward(ctx, g_out):
        rows, w, offsets = ctx.saved_tensors
        g_out = g_out.contiguous()
        g_rows = g_w = None
        if ctx.needs_input_grad[0]:
            # d rows = g_out @ w: the same grouped kernel on the transposed matrices
            g_rows = torch.zeros_like(rows)
            grouped_gemm_bf16(g_out, w.transpose(1, 2).contiguous(), offsets, out=g_rows, rows_hint=rows.shape[0])
        if ctx.needs_input_grad[1]:
            offs = offsets.tolist()
            g_w = torch.zeros_like(w)
            for e in range(w.shape[0]):
                lo, hi = offs[e], offs[e + 1]
                if hi > lo:
                    g_w[e] = g_out[lo:hi].t() @ rows[lo:hi]
        return g_rows, g_w, None


class MoELayer(nn.Module):
    def __init__(self, ep_comm, dim: int = 4096, ffn_dim: int = 1536, num_experts: int = 64, top_k: int = 8,
                 tokens_per_rank: int = 16384, capacity_factor: float = 2.0, device="cuda", seed: int = 0):
        super().__init__()
        self.comm, self.E, self.k, self.dim = ep_comm, num_experts, top_k, dim
        self.El = num_experts // ep_comm.nranks
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.router = nn.Parameter((torch.randn(num_experts, dim, generator=g) * 0.02).to(device=device, dtype=torch.bfloat16))
        base = ep_comm.rank * self.El
        ge = torch.Generator(device="cpu").manual_seed(seed + 1 + base)
        self.w13 = nn.Parameter((torch.randn(self.El, 2 * ffn_dim, dim, generator=ge) * 0.02).to(device=device, dtype=torch.bfloat16))
        self.w2 = nn.Parameter((torch.randn(self.El, dim, ffn_dim, generator=ge) * 0.02).to(device=device, dtype=torch.bfloat16))
        cap = int(capacity_factor * tokens_per_rank * top_k)
        self.dispatcher = MoeDispatcher(ep_comm, num_experts, dim, cap)
        self.ffn_dim = ffn_dim
        self.tokens_hint = tokens_per_rank * top_k
        self._w13_fused = None          # (version of w13, gate / up rows interleaved for the SwiGLU epilogue)
        self.last_dropped = None        # int32 [1] on the device: rows this rank could not take in the last forward

    def _fused_w13(self) -> torch.Tensor:
        v = self.w13._version
        if self._w13_fused is None or self._w13_fused[0] != v:
            self._w13_fused = (v, interleave_gate_up(self.w13.detach(), self.ffn_dim))
        return self._w13_fused[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = (x @ self.router.t()).float()
        top = logits.topk(self.k, dim=1)
        idx, w = top.indices.to(torch.int32), torch.softmax(top.values, dim=1)
        fusable = self.ffn_dim % 32 == 0 and x.is_cuda
        if torch.is_grad_enabled() and (x.requires_grad or self.w2.requires_grad):
            rows, offsets, send_pos = ep_dispatch(self.dispatcher, x, idx)
            h = GroupedLinear.apply(rows, self.w13, offsets)
            a = (F.silu(h[:, : self.ffn_dim].float()) * h[:, self.ffn_dim:].float()).to(torch.bfloat16)
            y = GroupedLinear.apply(a, self.w2, offsets)
            return ep_combine(self.dispatcher, y, w, idx, send_pos)
        res = self.dispatcher.dispatch(x.contiguous(), idx)
        self.last_dropped = res.dropped
        if fusable:
            a = grouped_gemm_bf16(res.recv_x, self._fused_w13(), res.expert_offsets, rows_hint=self.tokens_hint, swiglu=True)
        else:
            h = grouped_gemm_bf16(res.recv_x, self.w13.detach(), res.expert_offsets, rows_hint=self.tokens_hint)
            a = (F.silu(h[:, : self.ffn_dim].float()) * h[:, self.ffn_dim:].float()).to(torch.bfloat16)
        # the second GEMM writes the experts' outputs where the combine reads them
        grouped_gemm_bf16(a, self.w2.detach(), res.expert_offsets, out=self.dispatcher.y, rows_hint=self.tokens_hint)
        return self.dispatcher.combine(idx, w, res.send_pos)
