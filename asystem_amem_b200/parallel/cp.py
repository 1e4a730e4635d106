"""Context (sequence) parallel attention on the library's primitives.

The reference scales nothing along the sequence (it has no attention code at all); these two
wrappers show that the usual long-context schemes need no collective beyond the ones the
library already keeps alive across ncclPause / ncclResume:

* ``ulysses_attention``: the sequence is sharded over the ranks; one all-to-all turns the
  sequence shards of all heads into the full sequence of ``H / n`` heads, attention runs
  locally, a second all-to-all turns the result back (DeepSpeed-Ulysses formulation).
* ``ring_attention``: K/V blocks travel round the ring with grouped send/recv while every rank
  folds the block it holds into an online-softmax accumulator (blockwise / ring attention);
  with ``causal=True`` blocks that lie entirely in the future are skipped.

Both take and return ``[S_local, H, D]`` tensors (this rank's slice of the sequence) and work on
CUDA tensors (NVLink kernels) as well as on CPU tensors (mock backend), which is how they are
tested without a GPU.  The attention arithmetic itself is plain PyTorch.
"""
from __future__ import annotations

import math

import torch

from ..comm import group_end, group_start


def _seq_to_heads(comm, x: torch.Tensor) -> torch.Tensor:
    """[S_local, H, D] (all heads, my positions) -> [S, H / n, D] (my heads, all positions)."""
    n = comm.nranks
    s_local, heads, dim = x.shape
    send = x.reshape(s_local, n, heads // n, dim).permute(1, 0, 2, 3).contiguous()  # block j: head group j
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv)                                                     # block j: positions of rank j
    return recv.reshape(n * s_local, heads // n, dim)


def _heads_to_seq(comm, x: torch.Tensor, s_local: int) -> torch.Tensor:
    """Inverse of ``_seq_to_heads``."""
    n = comm.nranks
    _, heads_local, dim = x.shape
    send = x.reshape(n, s_local, heads_local, dim).contiguous()                      # block j: positions of rank j
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv)                                                     # block j: head group j
    return recv.permute(1, 0, 2, 3).reshape(s_local, n * heads_local, dim)


def _attend(q, k, v, causal: bool, q_offset: int = 0, k_offset: int = 0):
    """softmax(q k^T / sqrt(D) [+ causal mask]) v and the row-wise log-sum-exp, fp32 math.
    q: [Sq, H, D], k/v: [Sk, H, D]; offsets are the global positions of the first rows."""
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * scale
    if causal:
        qi = torch.arange(q.shape[0], device=q.device).unsqueeze(1) + q_offset
        ki = torch.arange(k.shape[0], device=q.device).unsqueeze(0) + k_offset
        s = s.masked_fill((ki > qi).unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                   # [H, Sq]
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)                                   # rows with no visible key
    out = torch.einsum("hqk,khd->qhd", p, v.float())
    return out, lse


def ulysses_attention(comm, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """Attention over the whole sequence for sequence-sharded q, k, v of shape [S_local, H, D];
    H must be divisible by the number of ranks.  Two all-to-alls per call (four tensors moved)."""
    n = comm.nranks
    s_local, heads, _ = q.shape
    if heads % n:
        raise ValueError(f"{heads} heads do not divide over {n} ranks")
    if n == 1:
        return _attend(q, k, v, causal)[0].to(q.dtype)
    qf, kf, vf = (_seq_to_heads(comm, t) for t in (q, k, v))
    out, _ = _attend(qf, kf, vf, causal)
    return _heads_to_seq(comm, out.to(q.dtype).contiguous(), s_local)


def ring_attention(comm, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """Blockwise attention with K/V travelling round the ring (grouped send/recv, one step per
    rank).  Partial results are merged with their log-sum-exp, so the outcome equals attention
    over the concatenated sequence up to fp32 rounding."""
    n, me = comm.nranks, comm.rank
    s_local = q.shape[0]
    acc = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse = torch.full((q.shape[1], s_local), float("-inf"), dtype=torch.float32, device=q.device)
    kv = torch.stack([k, v]).contiguous()
    nxt, prv = (me + 1) % n, (me - 1) % n
    for step in range(n):
        src = (me - step) % n                     # owner of the block held in this step
        if not causal or src <= me:
            part, part_lse = _attend(q, kv[0], kv[1], causal and src == me, me * s_local, src * s_local)
            new_lse = torch.logaddexp(lse, part_lse)
            w_old = torch.nan_to_num(torch.exp(lse - new_lse), nan=0.0).transpose(0, 1).unsqueeze(-1)
            w_new = torch.nan_to_num(torch.exp(part_lse - new_lse), nan=0.0).transpose(0, 1).unsqueeze(-1)
            acc = acc * w_old + part * w_new
            lse = new_lse
        if step + 1 < n:
            incoming = torch.empty_like(kv)
            group_start()
            comm.send(kv, nxt)
            comm.recv(incoming, prv)
            group_end()
            kv = incoming
    return acc.to(q.dtype)
