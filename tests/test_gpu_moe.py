"""MoE dispatch (permute fused into the all-to-all) and combine against a PyTorch reference."""
import pytest
import torch

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,E,k,T,d", [(2, 8, 2, 64, 64), (4, 16, 4, 300, 256), (4, 64, 8, 512, 128), (8, 64, 8, 129, 64)])
def test_dispatch_layout_and_combine(world, E, k, T, d):
    from asystem_amem_b200.ops import MoeDispatcher
    g = torch.Generator().manual_seed(world * 100 + E)
    xs = [torch.randn(T, d, generator=g).to(torch.bfloat16) for _ in range(world)]
    logits = [torch.randn(T, E, generator=g) for _ in range(world)]
    idx = [lg.topk(k, dim=1).indices.to(torch.int32) for lg in logits]
    ws = [torch.softmax(lg.topk(k, dim=1).values, dim=1) for lg in logits]
    El = E // world
    cap = world * T * k

    def fn(rank, world, comm, stream):
        disp = MoeDispatcher(comm, E, d, cap)
        outs = []
        for rep in range(2):
            res = disp.dispatch(xs[rank].cuda(), idx[rank].cuda())
            stream.synchronize()
            counts = res.expert_counts.cpu()
            offs = res.expert_offsets.cpu()
            total = int(offs[-1])
            recv = res.recv_x[:total].clone()
            # "expert" el multiplies its rows by (global expert id + 1) / 8
            y = disp.y
            for el in range(El):
                lo, hi = int(offs[el]), int(offs[el + 1])
                y[lo:hi] = (recv[lo:hi].float() * ((rank * El + el + 1) / 8.0)).to(torch.bfloat16)
            out = disp.combine(idx[rank].cuda(), ws[rank].cuda(), res.send_pos)
            stream.synchronize()
            outs.append((recv.cpu(), counts, out.cpu()))
        return outs

    res = run_emulated(world, fn)
    for rank, outs in enumerate(res):
        # expected receive layout: by local expert, then source rank, then (token, choice) order
        rows, exp_counts = [], []
        for el in range(El):
            e = rank * El + el
            c = 0
            for src in range(world):
                pairs = (idx[src].reshape(-1) == e).nonzero().flatten()
                rows.append(xs[src][pairs // k])
                c += len(pairs)
            exp_counts.append(c)
        exp_recv = torch.cat(rows)
        sel = idx[rank].long()
        scale = ((sel + 1).float() / 8.0)
        exp_out = ((xs[rank].float().unsqueeze(1) * scale.unsqueeze(2)).to(torch.bfloat16).float() * ws[rank].unsqueeze(2)).sum(1)
        for recv, counts, out in outs:
            assert counts.tolist() == exp_counts
            assert torch.equal(recv, exp_recv)
            torch.testing.assert_close(out.float(), exp_out, rtol=2e-2, atol=2e-2)
        assert torch.equal(outs[0][2], outs[1][2])


def _dense_reference(xs, idx, ws, W, G):
    """fp32 autograd reference of out[t] = sum_c w[t,c] * (x[t] @ W[idx[t,c]]), loss = sum(out * G)."""
    world = len(xs)
    Wr = W.clone().float().requires_grad_(True)
    grads = []
    for r in range(world):
        x = xs[r].float().requires_grad_(True)
        w = ws[r].clone().requires_grad_(True)
        sel = Wr[idx[r].long()]                                   # [T, k, d, d]
        y = torch.einsum("td,tkde->tke", x, sel)
        out = (y * w.unsqueeze(2)).sum(1)
        (out * G[r].float()).sum().backward()
        grads.append((out.detach(), x.grad, w.grad))
    return grads, Wr.grad


@pytest.mark.parametrize("world,E,k,T,d", [(2, 4, 2, 40, 64), (4, 16, 4, 96, 64)])
def test_expert_parallel_backward_steps(world, E, k, T, d):
    """The four forward / backward steps of parallel/ep.py, every rank a thread; the experts are
    one [d, d] matrix each and their local gradient comes from autograd on this rank's rows."""
    from asystem_amem_b200.ops import MoeDispatcher
    from asystem_amem_b200.parallel import ep
    g = torch.Generator().manual_seed(world * 10 + k)
    xs = [torch.randn(T, d, generator=g).to(torch.bfloat16) for _ in range(world)]
    logits = [torch.randn(T, E, generator=g) for _ in range(world)]
    idx = [lg.topk(k, dim=1).indices.to(torch.int32) for lg in logits]
    ws = [torch.softmax(lg.topk(k, dim=1).values, dim=1) for lg in logits]
    W = (torch.randn(E, d, d, generator=g) / d ** 0.5).to(torch.bfloat16)
    G = [torch.randn(T, d, generator=g).to(torch.bfloat16) for _ in range(world)]
    El = E // world

    def fn(rank, world, comm, stream):
        disp = MoeDispatcher(comm, E, d, world * T * k)
        x, ix, w = xs[rank].cuda(), idx[rank].cuda(), ws[rank].cuda()
        Wl = W[rank * El:(rank + 1) * El].cuda().float().requires_grad_(True)
        rows, offsets, send_pos, total = ep.dispatch_forward(disp, x, ix)
        offs = offsets.tolist()
        rows_leaf = rows.float().requires_grad_(True)
        y_rows = torch.cat([rows_leaf[offs[e]:offs[e + 1]] @ Wl[e] for e in range(El)]).to(torch.bfloat16)
        out = ep.combine_forward(disp, y_rows.detach(), ix, w, send_pos)
        g_y, g_w = ep.combine_backward(disp, G[rank].cuda(), y_rows.detach(), ix, w, send_pos)
        g_rows, g_W = torch.autograd.grad(y_rows, (rows_leaf, Wl), g_y)
        g_x = ep.dispatch_backward(disp, g_rows, ix, send_pos)
        stream.synchronize()
        return out.cpu(), g_x.cpu(), g_w.cpu(), g_W.cpu()

    res = run_emulated(world, fn)
    ref, ref_gW = _dense_reference(xs, idx, ws, W, G)
    for rank, (out, g_x, g_w, g_W) in enumerate(res):
        r_out, r_gx, r_gw = ref[rank]
        torch.testing.assert_close(out.float(), r_out, rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(g_x.float(), r_gx, rtol=5e-2, atol=5e-2)
        torch.testing.assert_close(g_w.float(), r_gw, rtol=5e-2, atol=8e-2)
        torch.testing.assert_close(g_W.float(), ref_gW[rank * El:(rank + 1) * El], rtol=5e-2, atol=1e-1)


def test_moe_layer_autograd_one_rank():
    """loss.backward() through the autograd wrappers (one rank: the engine's device thread runs
    the communication steps alone) against the same layer written densely in fp32."""
    import torch.nn.functional as F
    from asystem_amem_b200.models import MoELayer
    dim, ffn, E, k, T = 64, 32, 8, 2, 80
    g = torch.Generator().manual_seed(11)
    x0 = torch.randn(T, dim, generator=g).to(torch.bfloat16)
    G = torch.randn(T, dim, generator=g).to(torch.bfloat16)

    def fn(rank, world, comm, stream):
        layer = MoELayer(comm, dim, ffn, E, k, tokens_per_rank=T, capacity_factor=1.0, seed=3)
        x = x0.cuda().requires_grad_(True)
        out = layer(x)
        (out.float() * G.cuda().float()).sum().backward()
        stream.synchronize()
        return (out.detach().cpu(), x.grad.cpu(), layer.router.grad.cpu(), layer.w13.grad.cpu(), layer.w2.grad.cpu(),
                layer.router.detach().cpu(), layer.w13.detach().cpu(), layer.w2.detach().cpu())

    out, gx, g_router, g_w13, g_w2, router, w13, w2 = run_emulated(1, fn)[0]
    x = x0.float().requires_grad_(True)
    R, A, B2 = (t.float().requires_grad_(True) for t in (router, w13, w2))
    logits = x @ R.t()
    top = (x0 @ router.t()).float().topk(k, dim=1)          # same selection as the bf16 router matmul
    w = torch.softmax(logits.gather(1, top.indices), dim=1)
    h = torch.einsum("td,tkfd->tkf", x, A[top.indices])
    a = F.silu(h[..., :ffn]) * h[..., ffn:]
    y = torch.einsum("tkf,tkdf->tkd", a, B2[top.indices])
    ref = (y * w.unsqueeze(2)).sum(1)
    (ref * G.float()).sum().backward()
    torch.testing.assert_close(out.float(), ref.detach(), rtol=5e-2, atol=3e-2)
    torch.testing.assert_close(gx.float(), x.grad, rtol=8e-2, atol=5e-2)
    torch.testing.assert_close(g_w2.float(), B2.grad, rtol=8e-2, atol=5e-2)
    torch.testing.assert_close(g_w13.float(), A.grad, rtol=8e-2, atol=5e-2)
    torch.testing.assert_close(g_router.float(), R.grad, rtol=1e-1, atol=1e-1)


def test_capacity_overflow_is_a_result_not_an_error():
    """A rank that is routed more rows than its buffers hold keeps the head of the sequence and
    reports the rest as dropped; counts and offsets stay inside the buffer, the combine gives the
    dropped choices weight zero, and the communicator keeps working afterwards."""
    from asystem_amem_b200.ops import MoeDispatcher
    world, E, k, T, d = 4, 8, 2, 128, 64
    El = E // world
    g = torch.Generator().manual_seed(77)
    xs = [torch.randn(T, d, generator=g).to(torch.bfloat16) for _ in range(world)]
    # every token picks expert 0 (rank 0) and one other expert: rank 0 is routed world * T rows plus its share
    idx = [torch.stack([torch.zeros(T, dtype=torch.int64), torch.randint(1, E, (T,), generator=g)], 1).to(torch.int32) for _ in range(world)]
    ws = [torch.full((T, k), 0.5) for _ in range(world)]
    cap = T * k                                     # rank 0 is sent at least world * T = 2 * cap rows

    def fn(rank, world, comm, stream):
        disp = MoeDispatcher(comm, E, d, cap)
        res = disp.dispatch(xs[rank].cuda(), idx[rank].cuda())
        stream.synchronize()
        offs, counts = res.expert_offsets.cpu(), res.expert_counts.cpu()
        total = int(offs[-1])
        disp.y[:total] = res.recv_x[:total]          # identity experts
        out = disp.combine(idx[rank].cuda(), ws[rank].cuda(), res.send_pos)
        stream.synchronize()
        first = (int(res.dropped.item()), offs.tolist(), counts.tolist(), res.send_pos.cpu(), out.cpu(), comm.async_error())
        # the communicator is still usable: a collective and a second dispatch go through
        t = torch.full((1000,), float(rank + 1), device="cuda")
        comm.all_reduce(t)
        res2 = disp.dispatch(xs[rank].cuda(), idx[rank].cuda())
        stream.synchronize()
        return first, float(t[0].item()), torch.equal(res2.send_pos.cpu(), first[3])

    res = run_emulated(world, fn)
    routed = [0] * world
    for src in range(world):
        for e in idx[src].reshape(-1).tolist():
            routed[e // El] += 1
    for rank, (first, summed, again) in enumerate(res):
        dropped, offs, counts, send_pos, out, err = first
        assert err == 0 and summed == sum(range(1, world + 1)) and again
        assert dropped == max(0, routed[rank] - cap)
        assert offs[-1] == min(routed[rank], cap) and sum(counts) == offs[-1] and max(offs) <= cap
        # a dropped choice contributes nothing; a kept one contributes 0.5 * x
        kept = (send_pos >= 0).float()
        exp = (xs[rank].float().unsqueeze(1) * (0.5 * kept).unsqueeze(2)).sum(1)
        torch.testing.assert_close(out.float(), exp, rtol=2e-2, atol=2e-2)
    assert res[0][0][0] > 0                          # the case really overflowed rank 0
    # every choice that went to rank 0 beyond its capacity is marked on the sender
    lost = sum(int((r[0][3] < 0).sum()) for r in res)
    assert lost == sum(max(0, routed[r] - cap) for r in range(world))
