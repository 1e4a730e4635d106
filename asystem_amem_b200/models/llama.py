"""Llama-3-architecture decoder (RMSNorm, rotary embeddings, grouped-query attention, SwiGLU)
with random initialisation.  The math is plain PyTorch; the library's part is the
communication around it (see parallel.fsdp).

Reference parity: none -- the reference ships no model; this decoder is the workload of the
train / infer switching benchmark (the RL co-location scenario of README.md:1-60).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5

    @classmethod
    def llama3_8b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=256)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


def rope_tables(seq: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(seq, device=device).float(), inv)
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    # x: [B, H, S, D]
    x1, x2 = x.float()[..., 0::2], x.float()[..., 1::2]
    o1 = x1 * cos - x2 * sin
    o2 = x1 * sin + x2 * cos
    return torch.stack((o1, o2), dim=-1).flatten(-2).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.h, self.kv, self.hd = cfg.n_heads, cfg.n_kv_heads, cfg.dim // cfg.n_heads
        self.wq = nn.Linear(cfg.dim, cfg.n_heads * self.hd, bias=False)
        self.wk = nn.Linear(cfg.dim, cfg.n_kv_heads * self.hd, bias=False)
        self.wv = nn.Linear(cfg.dim, cfg.n_kv_heads * self.hd, bias=False)
        self.wo = nn.Linear(cfg.n_heads * self.hd, cfg.dim, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        q = self.wq(x).view(B, S, self.h, self.hd).transpose(1, 2)
        k = self.wk(x).view(B, S, self.kv, self.hd).transpose(1, 2)
        v = self.wv(x).view(B, S, self.kv, self.hd).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv != self.h)
        return self.wo(o.transpose(1, 2).reshape(B, S, -1))


class SwiGLU(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.w1 = nn.Linear(cfg.dim, cfg.ffn_dim, bias=False)
        self.w3 = nn.Linear(cfg.dim, cfg.ffn_dim, bias=False)
        self.w2 = nn.Linear(cfg.ffn_dim, cfg.dim, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attn_norm, self.attn = RMSNorm(cfg.dim, cfg.norm_eps), Attention(cfg)
        self.mlp_norm, self.mlp = RMSNorm(cfg.dim, cfg.norm_eps), SwiGLU(cfg)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.attn_norm(x), cos, sin)
        return x + self.mlp(self.mlp_norm(x))


class Embed(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.tok = nn.Embedding(cfg.vocab_size, cfg.dim)

    def forward(self, ids, cos=None, sin=None):
        return self.tok(ids)


class Head(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.out = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)

    def forward(self, x, cos=None, sin=None):
        return self.out(self.norm(x))


class LlamaDecoder(nn.Module):
    """units = [embedding, block_0 .. block_{L-1}, head]; each unit is one FSDP shard group."""

    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.cfg = cfg
        with torch.device(device):
            self.units = nn.ModuleList([Embed(cfg)] + [Block(cfg) for _ in range(cfg.n_layers)] + [Head(cfg)])
        self.to(dtype)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02)

    def forward(self, ids):
        cos, sin = rope_tables(ids.shape[1], self.cfg.dim // self.cfg.n_heads, self.cfg.rope_theta, ids.device)
        x = ids
        for u in self.units:
            x = u(x, cos, sin)
        return x

    def loss(self, ids, labels):
        logits = self.forward(ids)
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.view(-1))
