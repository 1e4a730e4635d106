#!/usr/bin/env python
"""Multi-GPU correctness run (one process per GPU; launch with torch.distributed.run).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 tests/multigpu_check.py

Checks, on real peer memory over NVLink: every collective against a PyTorch reference, the
all-reduce variants (one-shot, two-shot, NVLS when the multicast object could be built),
pause / resume cycles (memory really returned, results bit-identical), the fused
tensor-parallel GEMMs, the MoE dispatch / combine and a pipeline 1F1B step.  Prints one JSON line per check from
rank 0 and exits non-zero on the first failure.  NCCL (torch) is only used to cross-check.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asystem_amem_b200 import Communicator, NcclError, pause_all, resume_all  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = Communicator.from_torch_distributed()
    info = comm.info()
    failures = []

    def report(name, ok, **kw):
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(json.dumps({"check": name, "ok": bool(flag.item()), **kw}), flush=True)
        if not flag.item():
            failures.append(name)

    def gather_cpu(t):
        outs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(outs, t)
        return outs

    report("init", True, world=world, nvls=info["nvls"], emulated=info["emulated"], stage_mib=info["stage_bytes"] >> 20)

    # ---- all-reduce variants, several sizes and types
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1, 4097, 1 << 20, (1 << 24) + 40):
            g = torch.Generator().manual_seed(1000 + rank)
            x = torch.randn(n, generator=g).to(dtype)
            xs = gather_cpu(x)
            acc = xs[0].float()
            for t in xs[1:]:
                acc = acc + t.float()
            ref = acc.to(dtype)
            for algo in ("auto", "oneshot", "twoshot", "nvls"):
                if algo == "nvls" and not info["nvls"]:
                    continue
                if algo == "oneshot" and n * x.element_size() > (4 << 20):
                    continue
                y = x.cuda()
                try:
                    comm.all_reduce(y, algo=algo)
                except NcclError as e:
                    report(f"allreduce {dtype} n={n} {algo}", False, error=str(e))
                    continue
                torch.cuda.synchronize()
                if algo in ("nvls", "auto"):  # the switch's addition order is its own
                    ok = torch.allclose(y.cpu().float(), acc, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-2 if dtype == torch.bfloat16 else 1e-4)
                else:
                    ok = torch.equal(y.cpu(), ref)
                report(f"allreduce {str(dtype)[6:]} n={n} {algo}", ok)

    # ---- the other collectives
    n = 1 << 18
    x = (torch.arange(n, dtype=torch.float32) + rank * 1000).cuda()
    xs = gather_cpu(x.cpu())
    out = torch.empty(world * n, device="cuda")
    comm.all_gather(x, out)
    report("allgather", torch.equal(out.cpu(), torch.cat(xs)))
    send = torch.cat([x + 7 * j for j in range(world)])
    recv = torch.empty(n, device="cuda")
    comm.reduce_scatter(send, recv)
    exp = sum(t + 7 * rank for t in xs)
    report("reducescatter", torch.equal(recv.cpu(), exp))
    rb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    comm.reduce_scatter(send, rb, scale=1.0 / world)
    report("reducescatter scale+cast", torch.equal(rb.cpu(), (exp * (1.0 / world)).to(torch.bfloat16)))
    b = x.clone()
    comm.broadcast(b, root=world - 1)
    report("broadcast", torch.equal(b.cpu(), xs[world - 1]))
    r = torch.empty(n, device="cuda")
    comm.reduce(x, r, root=0)
    report("reduce", rank != 0 or torch.equal(r.cpu(), sum(xs)))
    s = torch.cat([torch.full((1000,), float(rank * 10 + j)) for j in range(world)]).cuda()
    t = torch.empty_like(s)
    comm.all_to_all(s, t)
    report("alltoall", torch.equal(t.cpu(), torch.cat([torch.full((1000,), float(j * 10 + rank)) for j in range(world)])))
    from asystem_amem_b200 import group_end, group_start
    sb, rcv = torch.full((1 << 22,), float(rank), device="cuda"), torch.empty(1 << 22, device="cuda")
    group_start()
    comm.send(sb, (rank + 1) % world)
    comm.recv(rcv, (rank - 1) % world)
    group_end()
    torch.cuda.synchronize()
    report("sendrecv ring 16MiB", bool((rcv == float((rank - 1) % world)).all()))

    # ---- messages of several chunks whose last chunk is short (device-generated integers: sums are exact)
    nb = 18_000_004                                   # 68.7 MiB of fp32 per rank: several chunks, an odd tail
    base = torch.arange(nb, device="cuda", dtype=torch.float32) % 1021
    mine_big = base + rank
    out_big = torch.empty(world * nb, device="cuda")
    comm.all_gather(mine_big, out_big)
    torch.cuda.synchronize()
    report("allgather, 69 MiB per rank", all(torch.equal(out_big[j * nb:(j + 1) * nb], base + j) for j in range(world)))
    send_big = torch.cat([base + rank + 3 * j for j in range(world)])
    comm.reduce_scatter(send_big, out_big[:nb])
    torch.cuda.synchronize()
    report("reducescatter, 69 MiB per rank", torch.equal(out_big[:nb], world * base + sum(range(world)) + 3 * rank * world))
    comm.all_to_all(send_big, out_big)
    torch.cuda.synchronize()
    report("alltoall, 69 MiB per peer", all(torch.equal(out_big[j * nb:(j + 1) * nb], base + j + 3 * rank) for j in range(world)))
    big = mine_big.repeat(3)[: 3 * nb - 5].contiguous()     # 206 MiB
    ref_big = (base * world + sum(range(world))).repeat(3)[: 3 * nb - 5]
    for algo in ("twoshot", "nvls") if info["nvls"] else ("twoshot",):
        for rep in range(3):
            yb = big.clone()
            comm.all_reduce(yb, algo=algo)
            torch.cuda.synchronize()
            report(f"allreduce 206 MiB fp32 {algo} #{rep}", torch.equal(yb, ref_big))
    bb = big.clone() if rank == 1 % world else torch.zeros_like(big)
    comm.broadcast(bb, root=1 % world)
    torch.cuda.synchronize()
    src_big = ((base + 1 % world).repeat(3))[: 3 * nb - 5]
    report("broadcast 206 MiB", torch.equal(bb, src_big))
    del out_big, send_big, big, ref_big, bb, src_big, mine_big, base
    torch.cuda.empty_cache()

    # ---- pause / resume: memory returns, same results afterwards, no re-init
    y0 = x.clone()
    comm.all_reduce(y0)
    torch.cuda.synchronize()
    dist.barrier()
    free0 = torch.cuda.mem_get_info()[0]
    ok, freed = True, 0
    for cycle in range(20):
        pause_all()
        freed = torch.cuda.mem_get_info()[0] - free0
        resume_all()
        y = x.clone()
        comm.all_reduce(y)
        torch.cuda.synchronize()
        ok = ok and torch.equal(y, y0)
    st = comm.pause_resume_stats()
    report("pause/resume x20", ok and freed >= 0.95 * info["stage_bytes"], freed_mib=freed >> 20,
           pause_ms=round(st["pause_total_us"] / 1e3, 3), resume_ms=round(st["resume_total_us"] / 1e3, 3))

    # ---- registered windows: in-place all-reduce (multicast when the communicator has NVLS), pause / resume
    for dtype, n in ((torch.bfloat16, (1 << 24) + 64), (torch.float32, 3_000_001)):
        es = torch.empty(0, dtype=dtype).element_size()
        win = comm.window_alloc(n * es + 4096)
        xw = win.tensor(dtype, n)
        g = torch.Generator().manual_seed(500 + rank)
        mine = torch.randn(n, generator=g).to(dtype)
        acc = sum(t.float() for t in gather_cpu(mine))
        xw.copy_(mine.cuda())
        torch.cuda.synchronize()
        dist.barrier()
        comm.all_reduce(xw, algo="window")
        torch.cuda.synchronize()
        first = xw.clone()
        ok = torch.allclose(first.cpu().float(), acc, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-2 if dtype == torch.bfloat16 else 1e-4)
        free_w = torch.cuda.mem_get_info()[0]
        for cycle in range(3):
            pause_all()
            freed_w = torch.cuda.mem_get_info()[0] - free_w
            resume_all()
            ok = ok and torch.equal(xw, first)               # the window's contents came back
            xw.copy_(mine.cuda())
            torch.cuda.synchronize()
            dist.barrier()
            comm.all_reduce(xw)                              # the tuner takes the window path
            torch.cuda.synchronize()
            ok = ok and torch.equal(xw, first)               # bit-identical to the run before the pause
        report(f"window allreduce {str(dtype)[6:]} n={n} + pause x3", ok and freed_w >= n * es, freed_mib=freed_w >> 20)
        win.free()

    # ---- reduce-scatter out of a window / all-gather into a window (multicast forms: three ranks or more)
    n_w = 1 << 20                                              # elements per rank
    win_s = comm.window_alloc(n_w * world * 4)
    win_r = comm.window_alloc(n_w * world * 4)
    src = win_s.tensor(torch.float32, n_w * world)
    g = torch.Generator().manual_seed(900 + rank)
    mine = torch.randn(n_w * world, generator=g)
    src.copy_(mine.cuda())
    torch.cuda.synchronize()
    dist.barrier()
    out_rs = torch.empty(n_w, device="cuda")
    comm.reduce_scatter(src, out_rs)
    torch.cuda.synchronize()
    exp = sum(t[rank * n_w:(rank + 1) * n_w] for t in gather_cpu(mine))
    report("reducescatter from a window", torch.allclose(out_rs.cpu(), exp, rtol=1e-5, atol=1e-4))
    dst = win_r.tensor(torch.float32, n_w * world)
    piece = (torch.arange(n_w, dtype=torch.float32) + 1000.0 * rank).cuda()
    comm.all_gather(piece, dst)
    torch.cuda.synchronize()
    report("allgather into a window", torch.equal(dst.cpu(), torch.cat(gather_cpu(piece.cpu()))))
    dist.barrier()
    win_r.free()
    win_s.free()

    # ---- fused tensor-parallel GEMMs
    from asystem_amem_b200.ops import MoeDispatcher, all_gather_gemm, gemm_reduce_scatter
    m_local, N, K = 512, 1024, 2048
    g = torch.Generator().manual_seed(7 + rank)
    a_shard = torch.randn(m_local, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    full = torch.cat(gather_cpu(a_shard)).float()
    outs = [all_gather_gemm(comm, a_shard.cuda(), w.cuda()).cpu() for _ in range(3)]
    ref = full @ w.float().t()
    ok = all((o.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2 for o in outs) and torch.equal(outs[0], outs[2])
    report("allgather->gemm", ok)
    act = torch.randn(m_local * world, K, generator=g).to(torch.bfloat16)
    part = act.float() @ w.float().t()
    parts = gather_cpu(part)
    exact = sum(p[rank * m_local:(rank + 1) * m_local] for p in parts)
    outs = [gemm_reduce_scatter(comm, act.cuda(), w.cuda()).cpu() for _ in range(3)]
    ok = all((o.float() - exact).abs().max().item() <= 3e-2 * exact.abs().max().item() + 2e-2 for o in outs) and torch.equal(outs[0], outs[2])
    report("gemm->reducescatter", ok)

    # ---- MoE dispatch / combine
    E, k, T, d = 8 * world, 4, 1024, 512
    xs_tok = torch.randn(T, d, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    top = logits.topk(k, dim=1)
    idx, wts = top.indices.to(torch.int32), torch.softmax(top.values, dim=1)
    disp = MoeDispatcher(comm, E, d, world * T * k)
    res = disp.dispatch(xs_tok.cuda(), idx.cuda())
    torch.cuda.synchronize()
    total = int(res.expert_offsets[-1].item())
    disp.y[:total] = res.recv_x[:total]  # identity experts
    out = disp.combine(idx.cuda(), wts.cuda(), res.send_pos)
    torch.cuda.synchronize()
    exp = (xs_tok.float().unsqueeze(1) * wts.unsqueeze(2)).sum(1)
    all_idx = gather_cpu(idx)
    El = E // world
    exp_total = sum(int(((i >= rank * El) & (i < (rank + 1) * El)).sum()) for i in all_idx)
    report("moe dispatch+combine", total == exp_total and torch.allclose(out.cpu().float(), exp, rtol=2e-2, atol=2e-2), rows=total)

    # ---- sharded data-parallel training steps on a tiny Llama, with and without a pause
    import torch.nn.functional as F
    from asystem_amem_b200.models import LlamaConfig, LlamaDecoder
    from asystem_amem_b200.models.llama import rope_tables
    from asystem_amem_b200.parallel import FSDP, ShardedAdamW
    cfg = LlamaConfig.tiny()

    def train(with_pause):
        torch.manual_seed(0)
        fsdp = FSDP(LlamaDecoder(cfg, device="cuda"), comm)
        opt = ShardedAdamW(fsdp, lr=1e-2)
        hist = []
        for step in range(3):
            ids = torch.randint(0, cfg.vocab_size, (2, 64), generator=torch.Generator().manual_seed(10 * step + rank)).cuda()
            cos, sin = rope_tables(64, cfg.dim // cfg.n_heads, cfg.rope_theta, "cuda")
            logits = fsdp.forward_units(ids, cos, sin)
            loss = F.cross_entropy(logits.float().view(-1, cfg.vocab_size), ids.view(-1))
            fsdp.zero_grad()
            loss.backward()
            hist.append((float(loss), float(fsdp.grad_norm())))
            opt.step()
            if with_pause:
                torch.cuda.synchronize()
                pause_all()
                resume_all()
        return hist

    h0, h1 = train(False), train(True)
    norms = gather_cpu(torch.tensor([h[1] for h in h0]))
    report("fsdp tiny llama, pause between steps", h0 == h1 and all(torch.equal(norms[0], t) for t in norms), losses=[round(h[0], 4) for h in h0])

    # ---- pipeline 1F1B over the library's send / recv (rendez-vous transfers: grouped exchanges)
    from asystem_amem_b200.parallel import PipelineStage
    torch.manual_seed(5)
    layers = [torch.nn.Linear(64, 64) for _ in range(world)]      # same on every rank (same seed)
    gp = torch.Generator().manual_seed(6)
    n_mb = 2 * world + 1
    mbs = [torch.randn(16, 64, generator=gp) for _ in range(n_mb)]
    tgt = [torch.randn(16, 64, generator=gp) for _ in range(n_mb)]
    mine = torch.nn.Linear(64, 64).cuda()
    mine.load_state_dict(layers[rank].state_dict())
    pipe = PipelineStage(comm, rank, world)
    losses = pipe.run_1f1b(lambda t: torch.tanh(mine(t)), [m.cuda() for m in mbs], torch.empty(16, 64, device="cuda"),
                           loss_fn=lambda y, i: ((y - tgt[i].cuda()) ** 2).mean())
    torch.cuda.synchronize()
    ref_losses = []
    for xb, tb in zip(mbs, tgt):
        hcur = xb
        for layer in layers:
            hcur = torch.tanh(layer(hcur))
        lref = ((hcur - tb) ** 2).mean()
        lref.backward()
        ref_losses.append(float(lref))
    ok = float((mine.weight.grad.cpu() - layers[rank].weight.grad).abs().max()) < 1e-4
    if rank == world - 1:
        ok = ok and all(abs(float(a) - b) < 1e-4 for a, b in zip(losses, ref_losses))
    report("pipeline 1F1B gradients equal the single-process run", ok, micro_batches=n_mb)

    err = comm.async_error()
    report("no device-side errors", err == 0)
    comm.destroy()
    dist.destroy_process_group()
    if failures:
        if rank == 0:
            print("FAILED:", failures, flush=True)
        sys.exit(1)
    if rank == 0:
        print("ALL OK", flush=True)


if __name__ == "__main__":
    main()
