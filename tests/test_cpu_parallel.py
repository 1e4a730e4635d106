"""CPU (mock backend) tests of the parallel wrappers: sharded data parallel training on a tiny
Llama decoder with a pause/resume between steps, and the pipeline-parallel forward schedule."""
import pytest
import torch

from mp_util import run_ranks


def _fsdp_train(rank, world, uid, with_pause):
    import torch
    from asystem_amem_b200 import Communicator, pause_all, resume_all
    from asystem_amem_b200.models import LlamaConfig, LlamaDecoder
    from asystem_amem_b200.parallel import FSDP, ShardedAdamW
    import torch.nn.functional as F
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny()
    model = LlamaDecoder(cfg, dtype=torch.bfloat16, device="cpu")
    comm = Communicator(world, rank, uid)
    fsdp = FSDP(model, comm)
    opt = ShardedAdamW(fsdp, lr=1e-2)
    from asystem_amem_b200.models.llama import rope_tables
    losses, norms = [], []
    for step in range(3):
        g = torch.Generator().manual_seed(100 * step + rank)
        ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
        cos, sin = rope_tables(16, cfg.dim // cfg.n_heads, cfg.rope_theta, "cpu")
        logits = fsdp.forward_units(ids, cos, sin)
        loss = F.cross_entropy(logits.float().view(-1, cfg.vocab_size), ids.view(-1))
        fsdp.zero_grad()
        loss.backward()
        norms.append(float(fsdp.grad_norm()))
        opt.step()
        losses.append(float(loss))
        if with_pause:
            pause_all()
            resume_all()
    comm.destroy()
    return losses, norms


def test_fsdp_tiny_llama_matches_with_and_without_pause():
    plain = run_ranks(_fsdp_train, 2, args=(False,), timeout=300)
    paused = run_ranks(_fsdp_train, 2, args=(True,), timeout=300)
    assert plain == paused                      # bitwise: pause/resume changes nothing
    for losses, norms in plain:
        assert all(torch.isfinite(torch.tensor(losses))) and norms[0] > 0
    assert plain[0][1] == plain[1][1]           # the global gradient norm is the same on every rank
    assert plain[0][0][2] < plain[0][0][0] + 1.0


def _fsdp_vs_dense(rank, world, uid):
    """Sharded gradients equal the average of the per-rank dense gradients."""
    import torch
    import torch.nn.functional as F
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.models import LlamaConfig, LlamaDecoder
    from asystem_amem_b200.models.llama import rope_tables
    from asystem_amem_b200.parallel import FSDP
    cfg = LlamaConfig.tiny()
    torch.manual_seed(0)
    dense = LlamaDecoder(cfg, dtype=torch.bfloat16, device="cpu")
    torch.manual_seed(0)
    model = LlamaDecoder(cfg, dtype=torch.bfloat16, device="cpu")
    comm = Communicator(world, rank, uid)
    fsdp = FSDP(model, comm)
    cos, sin = rope_tables(8, cfg.dim // cfg.n_heads, cfg.rope_theta, "cpu")
    grads = []
    for r in range(world):
        ids = torch.randint(0, cfg.vocab_size, (1, 8), generator=torch.Generator().manual_seed(r))
        dense.zero_grad()
        F.cross_entropy(dense(ids).float().view(-1, cfg.vocab_size), ids.view(-1)).backward()
        grads.append(torch.cat([p.grad.reshape(-1).float() for p in dense.units[1].parameters()]))
    ids = torch.randint(0, cfg.vocab_size, (1, 8), generator=torch.Generator().manual_seed(rank))
    logits = fsdp.forward_units(ids, cos, sin)
    F.cross_entropy(logits.float().view(-1, cfg.vocab_size), ids.view(-1)).backward()
    u = fsdp.units[1]
    ref = (sum(g.to(torch.bfloat16).float() for g in grads) / world)
    mine = u.grad_shard
    lo = rank * u.shard_len
    ref_shard = torch.zeros(u.shard_len)
    n = min(u.shard_len, ref.numel() - lo)
    ref_shard[:n] = ref[lo:lo + n]
    comm.destroy()
    return float((mine - ref_shard).abs().max()), float(ref_shard.abs().max())


def test_fsdp_gradients_match_dense_average():
    for err, scale in run_ranks(_fsdp_vs_dense, 2, timeout=300):
        assert err <= 2e-2 * scale + 1e-3, (err, scale)


def _pipeline(rank, world, uid):
    import torch
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.parallel import PipelineStage
    comm = Communicator(world, rank, uid)
    stage = PipelineStage(comm, rank, world)
    mbs = [torch.full((4, 8), float(i + 1)) for i in range(3)]
    outs = stage.run_gpipe(lambda x: x * 2 + rank, mbs, torch.empty(4, 8))
    comm.destroy()
    return None if outs is None else [float(o[0, 0]) for o in outs]


def test_pipeline_forward_schedule():
    res = run_ranks(_pipeline, 3)
    assert res[0] is None and res[1] is None
    # stage s computes 2x + s
    assert res[2] == [((2 * (i + 1) + 0) * 2 + 1) * 2 + 2 for i in range(3)]


def _pipeline_1f1b(rank, world, uid, n_mb=5):
    """One linear layer per stage, `n_mb` micro-batches: losses and every stage's accumulated
    weight gradient must equal those of the same layers run in one process."""
    import torch
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.parallel import PipelineStage
    comm = Communicator(world, rank, uid)
    torch.manual_seed(0)
    layers = [torch.nn.Linear(8, 8) for _ in range(world)]        # same on every rank (same seed)
    g = torch.Generator().manual_seed(1)
    mbs = [torch.randn(4, 8, generator=g) for _ in range(n_mb)]
    targets = [torch.randn(4, 8, generator=g) for _ in range(n_mb)]
    mine = layers[rank]
    stage = PipelineStage(comm, rank, world)
    losses = stage.run_1f1b(lambda x: torch.tanh(mine(x)), mbs, torch.empty(4, 8),
                            loss_fn=lambda y, i: ((y - targets[i]) ** 2).mean())
    got_grad = mine.weight.grad.clone()
    # reference: the whole pipeline in this process
    ref_layers = [torch.nn.Linear(8, 8) for _ in range(world)]
    for a, b in zip(ref_layers, layers):
        a.load_state_dict(b.state_dict())
    ref_losses = []
    for x, t in zip(mbs, targets):
        h = x
        for layer in ref_layers:
            h = torch.tanh(layer(h))
        loss = ((h - t) ** 2).mean()
        loss.backward()
        ref_losses.append(float(loss))
    comm.destroy()
    err = float((got_grad - ref_layers[rank].weight.grad).abs().max())
    return err, None if losses is None else [float(v) for v in losses], ref_losses


@pytest.mark.parametrize("stages,n_mb", [(3, 5), (4, 2), (2, 1), (4, 9)])
def test_pipeline_1f1b_matches_single_process_gradients(stages, n_mb):
    """More micro-batches than stages (a steady 1F1B phase), fewer (warm-up and drain only), one."""
    res = run_ranks(_pipeline_1f1b, stages, args=(n_mb,))
    for err, _losses, _ref in res:
        assert err < 1e-5, res
    assert all(r[1] is None for r in res[:-1])
    assert all(abs(a - b) < 1e-5 for a, b in zip(res[-1][1], res[-1][2])), res[-1]


def test_1f1b_plan_completes_under_rendezvous_semantics():
    """On the GPU a send completes only while the neighbour runs the matching receive.  Simulate
    that: every stage walks its plan in order, and a transfer step completes only when the
    neighbour's current step is its exact mirror (same micro-batches, both directions of a grouped
    exchange at once).  Every (stages, micro-batches) pair must run to the end."""
    from asystem_amem_b200.parallel.pp import plan_1f1b

    def ops(s, st):
        k = st[0]
        return {"recv_f": lambda: {("r", s - 1, "f", st[1])}, "send_f": lambda: {("s", s + 1, "f", st[1])},
                "recv_b": lambda: {("r", s + 1, "b", st[1])}, "send_b": lambda: {("s", s - 1, "b", st[1])},
                "send_f_recv_b": lambda: {("s", s + 1, "f", st[1]), ("r", s + 1, "b", st[2])},
                "send_b_recv_f": lambda: {("s", s - 1, "b", st[1]), ("r", s - 1, "f", st[2])}}[k]()

    for n in range(1, 7):
        for m in range(1, 13):
            plans = [[st for st in plan_1f1b(s, n, m) if st[0] not in ("fwd", "bwd")] for s in range(n)]
            for s in range(n):   # every micro-batch runs forward and backward exactly once, forward first
                order = [st for st in plan_1f1b(s, n, m) if st[0] in ("fwd", "bwd")]
                assert sorted(st[1] for st in order if st[0] == "fwd") == list(range(m))
                assert [st[1] for st in order if st[0] == "bwd"] == list(range(m))
                assert all(order.index(("fwd", i)) < order.index(("bwd", i)) for i in range(m))
            pos = [0] * n
            moved = True
            while moved:
                moved = False
                for s in range(n):
                    if pos[s] >= len(plans[s]):
                        continue
                    mine = ops(s, plans[s][pos[s]])
                    (q,) = {o[1] for o in mine}
                    if pos[q] >= len(plans[q]):
                        continue
                    mirror = {("r" if d == "s" else "s", s, t, i) for (d, _, t, i) in mine}
                    if mirror == ops(q, plans[q][pos[q]]):
                        pos[s] += 1
                        pos[q] += 1
                        moved = True
            assert all(pos[s] == len(plans[s]) for s in range(n)), (n, m, pos)


def test_1f1b_plan_keeps_at_most_n_minus_s_micro_batches_alive():
    """The point of 1F1B over GPipe: stage s never holds more than n - s forward results that
    still wait for their backward (GPipe would hold all m)."""
    from asystem_amem_b200.parallel.pp import plan_1f1b
    for n in range(1, 7):
        for m in range(1, 13):
            for s in range(n):
                alive = peak = 0
                for st in plan_1f1b(s, n, m):
                    if st[0] == "fwd":
                        alive += 1
                        peak = max(peak, alive)
                    elif st[0] == "bwd":
                        alive -= 1
                assert alive == 0 and peak <= min(m, n - s), (n, m, s, peak)


def _context_parallel(rank, world, uid, causal):
    import torch
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.parallel.cp import _attend, ring_attention, ulysses_attention
    comm = Communicator(world, rank, uid)
    s_local, heads, dim = 24, 2 * world, 16
    g = torch.Generator().manual_seed(3)
    full = [torch.randn(world * s_local, heads, dim, generator=g) for _ in range(3)]
    mine = [t[rank * s_local:(rank + 1) * s_local].contiguous() for t in full]
    ref = _attend(*full, causal)[0][rank * s_local:(rank + 1) * s_local]
    out_u = ulysses_attention(comm, *mine, causal=causal)
    out_r = ring_attention(comm, *mine, causal=causal)
    comm.destroy()
    return float((out_u - ref).abs().max()), float((out_r - ref).abs().max())


@pytest.mark.parametrize("world,causal", [(2, False), (3, True)])
def test_context_parallel_attention_matches_full_attention(world, causal):
    for err_ulysses, err_ring in run_ranks(_context_parallel, world, args=(causal,), timeout=300):
        assert err_ulysses < 1e-5 and err_ring < 1e-5, (err_ulysses, err_ring)


def _tp_mlp(rank, world, uid):
    """Column-parallel + row-parallel linears under sequence parallelism (host tensors: the
    composed form of the fused operations) against the dense computation, forward and backward."""
    import torch
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.parallel import ColumnParallelLinear, RowParallelLinear
    comm = Communicator(world, rank, uid)
    tokens, dim, ffn = 8 * world, 32, 16 * world
    g = torch.Generator().manual_seed(21)
    x = torch.randn(tokens, dim, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(ffn, dim, generator=g) * 0.2).to(torch.bfloat16)
    w2 = (torch.randn(dim, ffn, generator=g) * 0.2).to(torch.bfloat16)
    gout = torch.randn(tokens, dim, generator=g).to(torch.bfloat16)
    rows, fl = tokens // world, ffn // world
    col = ColumnParallelLinear(dim, ffn, comm, device="cpu")
    row = RowParallelLinear(ffn, dim, comm, device="cpu")
    with torch.no_grad():
        col.weight.copy_(w1[rank * fl:(rank + 1) * fl])
        row.weight.copy_(w2[:, rank * fl:(rank + 1) * fl])
    xs = x[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    y = row(torch.nn.functional.gelu(col(xs).float()).to(torch.bfloat16))
    y.backward(gout[rank * rows:(rank + 1) * rows])
    # dense reference in fp32 with the same bf16 rounding points
    xr = x.float().requires_grad_(True)
    w1r, w2r = w1.float().requires_grad_(True), w2.float().requires_grad_(True)
    h = torch.nn.functional.gelu((xr @ w1r.t()).to(torch.bfloat16).float()).to(torch.bfloat16).float()
    yr = h @ w2r.t()
    yr.backward(gout.float())
    sl = slice(rank * rows, (rank + 1) * rows)
    errs = (float((y.float() - yr[sl]).abs().max()), float((xs.grad.float() - xr.grad[sl]).abs().max()),
            float((col.weight.grad.float() - w1r.grad[rank * fl:(rank + 1) * fl]).abs().max()),
            float((row.weight.grad.float() - w2r.grad[:, rank * fl:(rank + 1) * fl]).abs().max()))
    comm.destroy()
    return errs


def test_tensor_parallel_layers_match_dense_on_host():
    for errs in run_ranks(_tp_mlp, 2, timeout=300):
        assert errs[0] < 0.03 and errs[1] < 0.03 and errs[2] < 0.08 and errs[3] < 0.08, errs   # bf16 rounding of outputs and gradients


def _expert_parallel(rank, world, uid):
    """loss.backward() through ep_dispatch / ep_combine with every rank a real process (host form
    of the dispatcher), against the dense computation out[t] = sum_c w[t,c] * (x[t] @ W[idx[t,c]])."""
    import torch
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.ops import MoeDispatcher
    from asystem_amem_b200.parallel.ep import ep_combine, ep_dispatch
    comm = Communicator(world, rank, uid)
    E, k, T, d = 2 * world, 2, 12, 16
    El = E // world
    g = torch.Generator().manual_seed(77)
    xs = [torch.randn(T, d, generator=g).to(torch.bfloat16) for _ in range(world)]
    logits = [torch.randn(T, E, generator=g) for _ in range(world)]
    W = (torch.randn(E, d, d, generator=g) / d ** 0.5)
    G = [torch.randn(T, d, generator=g).to(torch.bfloat16) for _ in range(world)]
    idx = [lg.topk(k, dim=1).indices.to(torch.int32) for lg in logits]
    disp = MoeDispatcher(comm, E, d, world * T * k)
    x = xs[rank].clone().requires_grad_(True)
    lg = logits[rank].clone().requires_grad_(True)
    w = torch.softmax(lg.gather(1, idx[rank].long()), dim=1)
    Wl = W[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    rows, offsets, send_pos = ep_dispatch(disp, x, idx[rank])
    offs = offsets.tolist()
    y_rows = torch.cat([(rows[offs[e]:offs[e + 1]].float() @ Wl[e]) for e in range(El)]).to(torch.bfloat16)
    out = ep_combine(disp, y_rows, w, idx[rank], send_pos)
    (out.float() * G[rank].float()).sum().backward()
    # dense reference
    Wr = W.clone().requires_grad_(True)
    ref = []
    for r in range(world):
        xr = xs[r].float().requires_grad_(True)
        lr = logits[r].clone().requires_grad_(True)
        wr = torch.softmax(lr.gather(1, idx[r].long()), dim=1)
        yr = torch.einsum("td,tkde->tke", xr, Wr[idx[r].long()])
        o = (yr * wr.unsqueeze(2)).sum(1)
        (o * G[r].float()).sum().backward()
        ref.append((o.detach(), xr.grad, lr.grad))
    errs = (float((out.float() - ref[rank][0]).abs().max()), float((x.grad.float() - ref[rank][1]).abs().max()),
            float((lg.grad - ref[rank][2]).abs().max()), float((Wl.grad - Wr.grad[rank * El:(rank + 1) * El]).abs().max()))
    comm.destroy()
    return errs


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_autograd_across_processes(world):
    for errs in run_ranks(_expert_parallel, world, timeout=300):
        assert errs[0] < 0.03 and errs[1] < 0.03 and errs[2] < 0.03 and errs[3] < 0.06, errs   # bf16 rounding


def _moe_layer(rank, world, uid):
    """The expert-parallel MoE layer (router, dispatch, SwiGLU experts, combine) trained one step
    per rank process on host tensors; compared with the same layer written densely."""
    import torch
    import torch.nn.functional as F
    from asystem_amem_b200 import Communicator
    from asystem_amem_b200.models import MoELayer
    comm = Communicator(world, rank, uid)
    dim, ffn, E, k, T = 32, 16, 2 * world, 2, 20
    layer = MoELayer(comm, dim, ffn, E, k, tokens_per_rank=T, capacity_factor=float(world), device="cpu", seed=5)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, dim, generator=g).to(torch.bfloat16).requires_grad_(True)
    G = torch.randn(T, dim, generator=g).to(torch.bfloat16)
    out = layer(x)
    (out.float() * G.float()).sum().backward()
    # every rank needs all experts' weights for the dense reference
    El = E // world
    w13_all = torch.empty(world * layer.w13.numel(), dtype=torch.bfloat16)
    w2_all = torch.empty(world * layer.w2.numel(), dtype=torch.bfloat16)
    comm.all_gather(layer.w13.detach().contiguous().view(-1), w13_all)
    comm.all_gather(layer.w2.detach().contiguous().view(-1), w2_all)
    A = w13_all.view(E, 2 * ffn, dim).float()
    B2 = w2_all.view(E, dim, ffn).float()
    xr = x.detach().float().requires_grad_(True)
    R = layer.router.detach().float().requires_grad_(True)
    top = (x.detach() @ layer.router.detach().t()).float().topk(k, dim=1)
    w = torch.softmax((xr @ R.t()).gather(1, top.indices), dim=1)
    h = torch.einsum("td,tkfd->tkf", xr, A[top.indices])
    a = F.silu(h[..., :ffn]) * h[..., ffn:]
    y = torch.einsum("tkf,tkdf->tkd", a, B2[top.indices])
    ref = (y * w.unsqueeze(2)).sum(1)
    (ref * G.float()).sum().backward()
    errs = (float((out.float() - ref.detach()).abs().max()), float((x.grad.float() - xr.grad).abs().max()),
            float((layer.router.grad.float() - R.grad).abs().max()))
    has_expert_grads = bool(layer.w13.grad is not None and layer.w2.grad is not None and layer.w2.grad.abs().sum() > 0)
    comm.destroy()
    return errs, has_expert_grads, El


def test_moe_layer_trains_across_processes_on_host():
    for errs, has_grads, _ in run_ranks(_moe_layer, 2, timeout=300):
        assert has_grads and errs[0] < 0.03 and errs[1] < 0.05 and errs[2] < 0.1, errs
