"""Expert-parallel MoE layer: top-k softmax routing, fused dispatch (permute inside the
all-to-all), per-expert SwiGLU FFN on the grouped rows, fused combine (un-permute + weighted
sum while pulling the rows back).  With gradients enabled the two communication steps run as
autograd functions whose backward passes reuse the same kernels (parallel/ep.py); under
``torch.no_grad()`` the experts write straight into the combine buffer and nothing is saved."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.moe import MoeDispatcher
from ..parallel.ep import ep_combine, ep_dispatch


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

    def _expert(self, el: int, rows: torch.Tensor) -> torch.Tensor:
        h = rows @ self.w13[el].t()
        a = (F.silu(h[:, : self.ffn_dim].float()) * h[:, self.ffn_dim:].float()).to(torch.bfloat16)
        return a @ self.w2[el].t()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = (x @ self.router.t()).float()
        top = logits.topk(self.k, dim=1)
        idx, w = top.indices.to(torch.int32), torch.softmax(top.values, dim=1)
        if torch.is_grad_enabled() and (x.requires_grad or self.w2.requires_grad):
            rows, offsets, send_pos = ep_dispatch(self.dispatcher, x, idx)
            offs = offsets.tolist()
            outs = [self._expert(el, rows[offs[el]:offs[el + 1]]) for el in range(self.El)]
            return ep_combine(self.dispatcher, torch.cat(outs), w, idx, send_pos)
        res = self.dispatcher.dispatch(x.contiguous(), idx)
        offs = res.expert_offsets.tolist()          # one host sync per layer: group boundaries
        y = self.dispatcher.y
        for el in range(self.El):
            lo, hi = offs[el], offs[el + 1]
            if hi > lo:
                y[lo:hi] = self._expert(el, res.recv_x[lo:hi])
        return self.dispatcher.combine(idx, w, res.send_pos)
