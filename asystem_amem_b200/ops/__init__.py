"""Fused operations: tcgen05 GEMM and its tensor-parallel forms, MoE dispatch/combine."""
from .gemm import all_gather_gemm, gemm_bf16, gemm_reduce_scatter, grouped_gemm_bf16, interleave_gate_up  # noqa: F401
from .moe import DispatchResult, MoeDispatcher  # noqa: F401,E402
