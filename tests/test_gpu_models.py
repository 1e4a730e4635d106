"""Model-level GPU tests on emulated ranks: tensor-parallel MLP (fused all-gather->GEMM and
GEMM->reduce-scatter, forward and backward) and the expert-parallel MoE layer, both against
dense PyTorch references.  (Sharded data-parallel training needs loss.backward(), whose
collectives would all run on the autograd engine's single per-device thread; it is covered by
the CPU rank processes in test_cpu_parallel.py and by tests/multigpu_check.py on real GPUs.)"""
import pytest
import torch
import torch.nn.functional as F

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_tp_mlp_forward_backward(world):
    from asystem_amem_b200.models import TPMLP
    dim, ffn, tokens = 256, 1024, 128 * world
    g = torch.Generator().manual_seed(3)
    x = torch.randn(tokens, dim, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(2 * ffn, dim, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(dim, ffn, generator=g) * 0.05).to(torch.bfloat16)
    gout = torch.randn(tokens, dim, generator=g).to(torch.bfloat16)
    fl = ffn // world

    def fn(rank, world, comm, stream):
        # Ranks are threads of one process here and PyTorch's autograd engine has ONE worker
        # thread per device, so the backward functions (which are collective) are called
        # directly instead of through loss.backward().
        from types import SimpleNamespace
        from asystem_amem_b200.parallel.tp import _ColumnFn, _RowFn
        mlp = TPMLP(comm, dim, ffn)
        with torch.no_grad():
            gate = w13[:ffn][rank * fl:(rank + 1) * fl]
            up = w13[ffn:][rank * fl:(rank + 1) * fl]
            mlp.w13.weight.copy_(torch.cat([gate, up]).cuda())
            mlp.w2.weight.copy_(w2[:, rank * fl:(rank + 1) * fl].cuda())
        rows = tokens // world
        xs = x[rank * rows:(rank + 1) * rows].cuda()
        with torch.no_grad():
            y = mlp(xs)
            h = mlp.w13(xs)
        hf = h.float().requires_grad_(True)
        act = (F.silu(hf[:, :fl]) * hf[:, fl:])
        act_b = act.detach().to(torch.bfloat16)
        gy = gout[rank * rows:(rank + 1) * rows].cuda()
        g_act, gw2, _ = _RowFn.backward(SimpleNamespace(comm=comm, saved_tensors=(act_b, mlp.w2.weight.detach())), gy)
        (gh,) = torch.autograd.grad(act, hf, g_act.float())      # elementwise only: no collective inside
        gx, gw13, _ = _ColumnFn.backward(SimpleNamespace(comm=comm, saved_tensors=(xs, mlp.w13.weight.detach())), gh.to(torch.bfloat16))
        stream.synchronize()
        return y.cpu(), gx.cpu(), gw2.cpu()

    res = run_emulated(world, fn)
    xr = x.float().requires_grad_(True)
    w13r, w2r = w13.float().requires_grad_(True), w2.float().requires_grad_(True)
    h = xr @ w13r.t()
    yr = (F.silu(h[:, :ffn]) * h[:, ffn:]) @ w2r.t()
    yr.backward(gout.float())
    rows = tokens // world
    for rank, (y, gx, gw2) in enumerate(res):
        sl = slice(rank * rows, (rank + 1) * rows)
        torch.testing.assert_close(y.float(), yr[sl].detach(), rtol=5e-2, atol=5e-2)
        torch.testing.assert_close(gx.float(), xr.grad[sl], rtol=8e-2, atol=8e-2)
        torch.testing.assert_close(gw2.float(), w2r.grad[:, rank * fl:(rank + 1) * fl], rtol=8e-2, atol=2e-1)


def test_moe_layer_matches_dense_reference():
    from asystem_amem_b200.models import MoELayer
    world, dim, ffn, E, k, T = 4, 128, 64, 16, 4, 96
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(T, dim, generator=g).to(torch.bfloat16) for _ in range(world)]

    def fn(rank, world, comm, stream):
        layer = MoELayer(comm, dim, ffn, E, k, tokens_per_rank=T, capacity_factor=float(world), seed=7)
        with torch.no_grad():
            out1 = layer(xs[rank].cuda())
            out2 = layer(xs[rank].cuda())
        stream.synchronize()
        return out1.cpu(), out2.cpu(), layer.router.detach().cpu(), layer.w13.detach().cpu(), layer.w2.detach().cpu()

    res = run_emulated(world, fn)
    router = res[0][2].float()
    w13 = torch.cat([r[3] for r in res]).float()   # [E, 2*ffn, dim]
    w2 = torch.cat([r[4] for r in res]).float()
    for rank, (o1, o2, *_rest) in enumerate(res):
        x = xs[rank]
        logits = (x @ router.to(torch.bfloat16).t()).float()
        top = logits.topk(k, dim=1)
        w = torch.softmax(top.values, dim=1)
        ref = torch.zeros(T, dim)
        for t in range(T):
            for j in range(k):
                e = int(top.indices[t, j])
                h = (x[t:t + 1] @ w13[e].to(torch.bfloat16).t())
                a = (F.silu(h[:, :ffn].float()) * h[:, ffn:].float()).to(torch.bfloat16)
                ref[t] += w[t, j] * (a @ w2[e].to(torch.bfloat16).t()).float()[0]
        torch.testing.assert_close(o1.float(), ref, rtol=5e-2, atol=2e-2)
        assert torch.equal(o1, o2)


@pytest.mark.parametrize("world,causal", [(2, True), (4, False)])
def test_context_parallel_attention_on_gpu(world, causal):
    """Ulysses (all-to-all) and ring (send/recv) attention over sequence shards against attention
    over the whole sequence, fp32."""
    from asystem_amem_b200.parallel.cp import _attend, ring_attention, ulysses_attention
    s_local, heads, dim = 64, 8, 32
    g = torch.Generator().manual_seed(9)
    full = [torch.randn(world * s_local, heads, dim, generator=g) for _ in range(3)]
    ref = _attend(*full, causal)[0]

    def fn(rank, world, comm, stream):
        mine = [t[rank * s_local:(rank + 1) * s_local].contiguous().cuda() for t in full]
        out_u = ulysses_attention(comm, *mine, causal=causal)
        out_r = ring_attention(comm, *mine, causal=causal)
        stream.synchronize()
        return out_u.cpu(), out_r.cpu()

    for rank, (out_u, out_r) in enumerate(run_emulated(world, fn)):
        sl = slice(rank * s_local, (rank + 1) * s_local)
        torch.testing.assert_close(out_u, ref[sl], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(out_r, ref[sl], rtol=1e-4, atol=1e-4)
