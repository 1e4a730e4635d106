"""Tensor-core GEMMs of the library (hand-written tcgen05 / TMEM / TMA kernels).

All take bf16 CUDA tensors with K contiguous: ``a`` is [M, K] (activations), ``b`` is [N, K]
(a ``torch.nn.Linear`` weight), the result is [M, N] = a @ b.T in bf16 with fp32 accumulation.

Reference parity: none -- the reference contains no GEMM and no fused operator (its plugin is
host code only, amem_nccl_plugin/Makefile:36).
"""
from __future__ import annotations

import torch

from .. import bindings as B


def _check(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("bf16 tensors expected")
    if not (a.is_cuda and b.is_cuda and a.is_contiguous() and b.is_contiguous()):
        raise ValueError("contiguous CUDA tensors expected")
    if a.shape[-1] != b.shape[-1]:
        raise ValueError(f"inner dimensions differ: {tuple(a.shape)} vs {tuple(b.shape)}")


def _on_host(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Host tensors (mock backend, no GPU): the operation is composed from the library's
    collective and a PyTorch matmul with fp32 accumulation, so that the parallel wrappers can be
    tested without a GPU.  CUDA tensors never take this path: they go to the tcgen05 kernels or
    fail."""
    return not a.is_cuda and not b.is_cuda


def _host_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a.float() @ b.float().t()


def _stream(stream) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ b[N, K].T on one GPU."""
    if _on_host(a, b):
        res = _host_matmul(a, b).to(a.dtype)
        return res if out is None else out.copy_(res)
    _check(a, b)
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device) if out is None else out
    lib = B.load_library()
    B.check(lib.amemGemmBf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, _stream(stream)), "amemGemmBf16")
    return out


def interleave_gate_up(w13: torch.Tensor, ffn: int) -> torch.Tensor:
    """[..., 2 * ffn, K] with the gate rows first and the up rows second  ->  the same rows in
    alternating blocks of 32 gate rows and 32 up rows, the layout the SwiGLU epilogue of
    :func:`grouped_gemm_bf16` expects (a column tile then holds a gate block next to its up
    block).  ``ffn`` must be a multiple of 32.  Done once per weight, not per step."""
    if ffn % 32 or w13.shape[-2] != 2 * ffn:
        raise ValueError("ffn must be a multiple of 32 and w13 must have 2 * ffn rows")
    lead, K = w13.shape[:-2], w13.shape[-1]
    gate = w13[..., :ffn, :].reshape(*lead, ffn // 32, 1, 32, K)
    up = w13[..., ffn:, :].reshape(*lead, ffn // 32, 1, 32, K)
    return torch.cat([gate, up], dim=-3).reshape(*lead, 2 * ffn, K).contiguous()


def grouped_gemm_bf16(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor | None = None,
                      rows_hint: int | None = None, swiglu: bool = False, stream=None) -> torch.Tensor:
    """For every group e: out[offsets[e]:offsets[e+1]] = a[offsets[e]:offsets[e+1]] @ w[e].T, in ONE
    launch of the tcgen05 kernel.  ``a`` is bf16 [rows_cap, K]; ``w`` is bf16 [groups, N, K];
    ``offsets`` is an int32 CUDA tensor of groups + 1 row offsets that stays on the device (the
    MoE dispatch's ``expert_offsets``: no host synchronisation).  Rows outside every group are
    left untouched.  With ``swiglu`` the rows of each ``w[e]`` must be in the layout of
    :func:`interleave_gate_up` and the result has N / 2 columns: silu(gate) * up, computed in the
    epilogue on the fp32 accumulators."""
    if not a.is_cuda:
        offs = offsets.tolist()
        N = w.shape[1]
        res = torch.zeros(a.shape[0], N // 2 if swiglu else N, dtype=a.dtype) if out is None else out
        for e in range(w.shape[0]):
            h = a[offs[e]:offs[e + 1]].float() @ w[e].float().t()
            if swiglu:
                h = h.view(h.shape[0], N // 64, 2, 32)
                h = (torch.nn.functional.silu(h[:, :, 0]) * h[:, :, 1]).reshape(h.shape[0], N // 2)
            res[offs[e]:offs[e + 1]] = h.to(a.dtype)
        return res
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or offsets.dtype != torch.int32:
        raise TypeError("bf16 operands and int32 offsets expected")
    if not (w.is_cuda and offsets.is_cuda and a.is_contiguous() and w.is_contiguous() and offsets.is_contiguous()):
        raise ValueError("contiguous CUDA tensors expected")
    groups, N, K = w.shape
    if a.shape[1] != K or offsets.numel() != groups + 1:
        raise ValueError(f"shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, {offsets.numel()} offsets")
    rows_cap = a.shape[0]
    out = torch.empty(rows_cap, N // 2 if swiglu else N, dtype=torch.bfloat16, device=a.device) if out is None else out
    lib = B.load_library()
    B.check(lib.amemGroupedGemmBf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), offsets.data_ptr(), groups, rows_cap,
                                    int(rows_hint or 0), N, K, 1 if swiglu else 0, _stream(stream)), "amemGroupedGemmBf16")
    return out


def all_gather_gemm(comm, a_shard: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """out[M, N] = all_gather_rows(a_shard)[M, K] @ b[N, K].T in ONE kernel (column-parallel
    linear under sequence parallelism).  ``a_shard`` holds this rank's M / nranks rows."""
    if _on_host(a_shard, b):
        full = torch.empty(a_shard.shape[0] * comm.nranks, a_shard.shape[1], dtype=a_shard.dtype)
        comm.all_gather(a_shard.contiguous(), full)
        res = _host_matmul(full, b).to(a_shard.dtype)
        return res if out is None else out.copy_(res)
    _check(a_shard, b)
    m_local, K = a_shard.shape
    M, N = m_local * comm.nranks, b.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a_shard.device) if out is None else out
    B.check(comm.lib.amemAllGatherGemm(a_shard.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, comm._h, _stream(stream)),
            "amemAllGatherGemm")
    return out


def gemm_reduce_scatter(comm, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """out[M / nranks, N] = reduce_scatter_rows(a[M, K_local] @ b[N, K_local].T) in ONE kernel
    (row-parallel linear under sequence parallelism)."""
    if _on_host(a, b):
        part = _host_matmul(a, b).contiguous()                     # fp32 partial products
        res32 = torch.empty(a.shape[0] // comm.nranks, b.shape[0], dtype=torch.float32)
        comm.reduce_scatter(part, res32)
        res = res32.to(a.dtype)
        return res if out is None else out.copy_(res)
    _check(a, b)
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty(M // comm.nranks, N, dtype=torch.bfloat16, device=a.device) if out is None else out
    B.check(comm.lib.amemGemmReduceScatter(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, comm._h, _stream(stream)),
            "amemGemmReduceScatter")
    return out
