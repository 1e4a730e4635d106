"""Tensor parallelism with sequence parallelism (Megatron style) on the fused GEMM kernels.

Activations between the two linears of a block are sharded by rows (tokens).  The
column-parallel linear all-gathers them inside its GEMM kernel; the row-parallel linear
reduce-scatters its output from the GEMM epilogue.  Backward uses the mirrored fused kernels
for the activation gradients and the library's own tcgen05 GEMM for the weight gradients.

Reference parity: none to match -- tensor parallelism appears in the reference only as
integration text (README.md:279-293, SGLang's tensor-model-parallel group); its users run
cuBLAS and NCCL back to back.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.gemm import all_gather_gemm, gemm_bf16, gemm_reduce_scatter


def _wgrad(gy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """gw[N, K] = gy[M, N].T @ x[M, K] on the library's tcgen05 GEMM, whose operands are both
    K-major: A = gy.T [N, M], B = x.T [K, M] (two transposing copies, then one tensor-core pass
    with fp32 accumulation over the M tokens).  Token counts that are not a multiple of 8 (the
    16-byte row rule of the TMA loads) fall back to a PyTorch matmul."""
    if gy.is_cuda and gy.shape[0] % 8 == 0 and gy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
        return gemm_bf16(gy.t().contiguous(), x.t().contiguous())
    return gy.t() @ x


class _ColumnFn(torch.autograd.Function):
    """y[M, N_local] = all_gather_rows(x_shard)[M, K] @ w[N_local, K].T"""

    @staticmethod
    def forward(ctx, x_shard, w, comm):
        ctx.comm = comm
        ctx.save_for_backward(x_shard, w)
        return all_gather_gemm(comm, x_shard.contiguous(), w.contiguous())

    @staticmethod
    def backward(ctx, gy):
        comm = ctx.comm
        x_shard, w = ctx.saved_tensors
        gy = gy.contiguous()
        # dx_shard = reduce_scatter_rows(gy @ w): the mirrored fused kernel, B = w.T [K, N_local]
        gx = gemm_reduce_scatter(comm, gy, w.t().contiguous())
        x_full = torch.empty(x_shard.shape[0] * comm.nranks, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        comm.all_gather(x_shard.contiguous(), x_full)
        gw = _wgrad(gy, x_full)
        return gx, gw, None


class _RowFn(torch.autograd.Function):
    """y_shard[M / n, N] = reduce_scatter_rows(x[M, K_local] @ w[N, K_local].T)"""

    @staticmethod
    def forward(ctx, x, w, comm):
        ctx.comm = comm
        ctx.save_for_backward(x, w)
        return gemm_reduce_scatter(comm, x.contiguous(), w.contiguous())

    @staticmethod
    def backward(ctx, gy_shard):
        comm = ctx.comm
        x, w = ctx.saved_tensors
        gy_shard = gy_shard.contiguous()
        # dx = all_gather_rows(gy_shard) @ w  -> fused all-gather GEMM with B = w.T [K_local, N]
        gx = all_gather_gemm(comm, gy_shard, w.t().contiguous())
        gy_full = torch.empty(gy_shard.shape[0] * comm.nranks, gy_shard.shape[1], dtype=gy_shard.dtype, device=gy_shard.device)
        comm.all_gather(gy_shard, gy_full)
        gw = _wgrad(gy_full, x)
        return gx, gw, None


class ColumnParallelLinear(nn.Module):
    """Weight [out_features / tp, in_features]; input rows sharded over the TP group."""

    def __init__(self, in_features: int, out_features: int, comm, device="cuda", std: float = 0.02):
        super().__init__()
        assert out_features % comm.nranks == 0
        self.comm = comm
        self.weight = nn.Parameter(torch.randn(out_features // comm.nranks, in_features, device=device, dtype=torch.bfloat16) * std)

    def forward(self, x_shard):
        return _ColumnFn.apply(x_shard, self.weight, self.comm)


class RowParallelLinear(nn.Module):
    """Weight [out_features, in_features / tp]; output rows sharded over the TP group."""

    def __init__(self, in_features: int, out_features: int, comm, device="cuda", std: float = 0.02):
        super().__init__()
        assert in_features % comm.nranks == 0
        self.comm = comm
        self.weight = nn.Parameter(torch.randn(out_features, in_features // comm.nranks, device=device, dtype=torch.bfloat16) * std)

    def forward(self, x):
        return _RowFn.apply(x, self.weight, self.comm)
