#!/usr/bin/env python
"""RL co-location cycle: training and inference share the GPUs and trade communicator memory.

One process per GPU holds TWO communicators over the same ranks: a training communicator
(sharded data-parallel Llama-3-8B-architecture step, seq 4096, micro-batch 1 per GPU, fused
gradient reduce-scatter + parameter all-gather) and an inference communicator (tensor-parallel,
sequence-parallel forward of a 64 x 2048-token random-id batch on the fused kernels: every
projection is one all-gather -> GEMM or one GEMM -> reduce-scatter launch).  The cycle is

    train step -> pause(train comm) -> TP inference batch -> pause(infer comm) -> resume(train comm)
    -> (next cycle) ... resume(infer comm) before its next use

and the script reports, as max over ranks, the switch latencies and the device memory each pause
returns.  `--layers` shrinks the model for small boxes (default: the full 32 layers).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29550 bench/rl_cycle.py --cycles 10

Reference parity: the use case the reference is built for (README.md:1-60, 'offload + reload <
1 s per step'): two process groups share the GPUs and take turns.
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator  # noqa: E402
from asystem_amem_b200.models import LlamaConfig, LlamaDecoder  # noqa: E402
from asystem_amem_b200.models.llama import RMSNorm, apply_rope, rope_tables  # noqa: E402
from asystem_amem_b200.ops import all_gather_gemm, gemm_reduce_scatter  # noqa: E402
from asystem_amem_b200.parallel import FSDP, ShardedAdamW  # noqa: E402


class TPInferenceLlama:
    """Tensor-parallel forward (prefill) with weights created directly in sharded form."""

    def __init__(self, cfg: LlamaConfig, comm, seed: int):
        n, r = comm.nranks, comm.rank
        self.cfg, self.comm = cfg, comm
        self.h, self.kv, self.hd = cfg.n_heads // n, max(1, cfg.n_kv_heads // n), cfg.dim // cfg.n_heads
        g = torch.Generator(device="cuda").manual_seed(seed + r)

        def w(*shape):
            return (torch.randn(*shape, device="cuda", generator=g) * 0.02).to(torch.bfloat16)

        self.embed = w(cfg.vocab_size, cfg.dim)
        self.layers = []
        for _ in range(cfg.n_layers):
            self.layers.append(dict(
                an=RMSNorm(cfg.dim, cfg.norm_eps).cuda().bfloat16(), mn=RMSNorm(cfg.dim, cfg.norm_eps).cuda().bfloat16(),
                wqkv=w((self.h + 2 * self.kv) * self.hd, cfg.dim), wo=w(cfg.dim, self.h * self.hd),
                w13=w(2 * (cfg.ffn_dim // n), cfg.dim), w2=w(cfg.dim, cfg.ffn_dim // n)))

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, chunk: int = 8) -> torch.Tensor:
        """ids [B, S]; sequences are processed `chunk` at a time to bound activation memory.
        Activations between the blocks are sharded by token rows (sequence parallel): every
        projection into a block is ONE all-gather -> GEMM kernel, every projection out of it ONE
        GEMM -> reduce-scatter kernel; no separate collective is launched."""
        cfg, comm = self.cfg, self.comm
        n, r = comm.nranks, comm.rank
        cos, sin = rope_tables(ids.shape[1], self.hd, cfg.rope_theta, ids.device)
        outs = []
        for b0 in range(0, ids.shape[0], chunk):
            sub = ids[b0:b0 + chunk]
            B, S = sub.shape
            T = B * S
            assert T % n == 0
            rows = T // n
            x = self.embed[sub.reshape(-1)[r * rows:(r + 1) * rows]]           # my token rows [T / n, d]
            for L in self.layers:
                hN = L["an"](x)
                qkv = all_gather_gemm(comm, hN.contiguous(), L["wqkv"])          # [T, (h + 2 kv) * hd] for my heads
                q, k, v = qkv.split([self.h * self.hd, self.kv * self.hd, self.kv * self.hd], dim=1)
                q = q.reshape(B, S, self.h, self.hd).transpose(1, 2)
                k = k.reshape(B, S, self.kv, self.hd).transpose(1, 2)
                v = v.reshape(B, S, self.kv, self.hd).transpose(1, 2)
                q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv != self.h)
                x = x + gemm_reduce_scatter(comm, o.transpose(1, 2).reshape(T, -1).contiguous(), L["wo"])
                hN = L["mn"](x)
                h13 = all_gather_gemm(comm, hN.contiguous(), L["w13"])           # gate | up for my slice of the FFN
                f = h13.shape[1] // 2
                act = (F.silu(h13[:, :f].float()) * h13[:, f:].float()).to(torch.bfloat16)
                x = x + gemm_reduce_scatter(comm, act, L["w2"])
            outs.append(x.float().mean())
        score = torch.stack(outs).mean().reshape(1)
        comm.all_reduce(score)
        return score[0] / n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--infer-batch", type=int, default=64)
    ap.add_argument("--infer-seq", type=int, default=2048)
    ap.add_argument("--cycles", type=int, default=10)
    ap.add_argument("--out", default="bench_results/rl_cycle.jsonl")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    train_comm = Communicator.from_torch_distributed()
    infer_comm = Communicator.from_torch_distributed()
    cfg = LlamaConfig.llama3_8b()
    cfg.n_layers = args.layers
    torch.manual_seed(0)
    fsdp = FSDP(LlamaDecoder(cfg, device="cuda"), train_comm)
    opt = ShardedAdamW(fsdp, lr=1e-5)
    infer = TPInferenceLlama(cfg, infer_comm, seed=1234)
    torch.cuda.synchronize()

    def mx(v):
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows = []
    infer_paused = False
    for c in range(args.cycles):
        ids = torch.randint(0, cfg.vocab_size, (1, args.seq), generator=torch.Generator().manual_seed(1000 * c + rank)).cuda()
        cos, sin = rope_tables(args.seq, cfg.dim // cfg.n_heads, cfg.rope_theta, "cuda")
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        logits = fsdp.forward_units(ids, cos, sin)
        loss = F.cross_entropy(logits.float().view(-1, cfg.vocab_size), ids.view(-1))
        fsdp.zero_grad()
        loss.backward()
        gn = fsdp.grad_norm()
        opt.step()
        torch.cuda.synchronize()
        t_train = time.perf_counter() - t0
        del logits
        f0 = torch.cuda.mem_get_info()[0]
        t0 = time.perf_counter()
        train_comm.pause()
        t_pause_train = time.perf_counter() - t0
        freed_train = torch.cuda.mem_get_info()[0] - f0
        t0 = time.perf_counter()
        if infer_paused:
            infer_comm.resume()
        t_resume_infer = time.perf_counter() - t0
        prompts = torch.randint(0, cfg.vocab_size, (args.infer_batch, args.infer_seq), generator=torch.Generator().manual_seed(c)).cuda()
        t0 = time.perf_counter()
        score = infer.prefill(prompts)
        torch.cuda.synchronize()
        t_infer = time.perf_counter() - t0
        f0 = torch.cuda.mem_get_info()[0]
        t0 = time.perf_counter()
        infer_comm.pause()
        infer_paused = True
        t_pause_infer = time.perf_counter() - t0
        freed_infer = torch.cuda.mem_get_info()[0] - f0
        t0 = time.perf_counter()
        train_comm.resume()
        t_resume_train = time.perf_counter() - t0
        row = {"cycle": c, "n_gpus": world, "layers": cfg.n_layers, "loss": round(float(loss), 4), "grad_norm": round(float(gn), 4),
               "infer_score": round(float(score), 5),
               "train_step_s": round(mx(t_train), 3), "infer_batch_s": round(mx(t_infer), 3),
               "pause_train_ms": round(mx(t_pause_train) * 1e3, 3), "resume_train_ms": round(mx(t_resume_train) * 1e3, 3),
               "pause_infer_ms": round(mx(t_pause_infer) * 1e3, 3), "resume_infer_ms": round(mx(t_resume_infer) * 1e3, 3),
               "switch_train_to_infer_ms": round(mx(t_pause_train + t_resume_infer) * 1e3, 3),
               "switch_infer_to_train_ms": round(mx(t_pause_infer + t_resume_train) * 1e3, 3),
               "gib_freed_pause_train": round(freed_train / 2**30, 4), "gib_freed_pause_infer": round(freed_infer / 2**30, 4)}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "a") as f:
                f.write(json.dumps(row) + "\n")
    infer_comm.resume()
    errs = train_comm.async_error() + infer_comm.async_error()
    if rank == 0:
        print(json.dumps({"device_errors": errs}), flush=True)
    dist.barrier()
    infer_comm.destroy()
    train_comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
