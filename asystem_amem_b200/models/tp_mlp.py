"""Tensor-parallel SwiGLU MLP block (Llama-3-70B shape by default: d=8192, ffn=28672) with
sequence-parallel activations: all-gather -> GEMM for the gate/up projection, GEMM ->
reduce-scatter for the down projection, both single fused kernels.

Reference parity: none -- the reference ships no model and no GEMM; baseline for these layers
is cuBLAS + NCCL.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel.tp import ColumnParallelLinear, RowParallelLinear


class TPMLP(nn.Module):
    def __init__(self, comm, dim: int = 8192, ffn_dim: int = 28672, device="cuda"):
        super().__init__()
        self.comm, self.ffn_local = comm, ffn_dim // comm.nranks
        # gate and up projections share one column-parallel GEMM: rows [0, ffn_local) = gate
        self.w13 = ColumnParallelLinear(dim, 2 * ffn_dim, comm, device=device)
        self.w2 = RowParallelLinear(ffn_dim, dim, comm, device=device)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """x_shard: bf16 [tokens / tp, dim] -> bf16 [tokens / tp, dim]"""
        h = self.w13(x_shard)
        gate, up = h[:, : self.ffn_local], h[:, self.ffn_local:]
        return self.w2((F.silu(gate.float()) * up.float()).to(torch.bfloat16))
