"""Test models: Llama-style decoder, tensor-parallel MLP block, expert-parallel MoE layer."""
from .llama import LlamaConfig, LlamaDecoder  # noqa: F401
from .moe_layer import MoELayer  # noqa: F401
from .tp_mlp import TPMLP  # noqa: F401
