"""GPU numerics of the collective kernels against plain PyTorch fp32 references.
Ranks run as threads on cuda:0 (emulated communicator, one cooperative grid per collective)."""
import pytest
import torch

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


def _inputs(world, n, dtype, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn(n, generator=g, dtype=torch.float32).to(dtype) for _ in range(world)]


def _ordered_sum(xs, out_dtype):
    acc = xs[0].float().clone()
    for x in xs[1:]:
        acc = acc + x.float()
    return acc.to(out_dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,algo", [(1, "auto"), (4097, "oneshot"), (4097, "twoshot"), (3 * 1024 * 1024 + 5, "twoshot")])
def test_allreduce(world, dtype, n, algo):
    xs = _inputs(world, n, dtype)
    ref = _ordered_sum(xs, dtype)

    def fn(rank, world, comm, stream):
        x = xs[rank].cuda()
        comm.all_reduce(x, algo=algo)
        y = xs[rank].cuda()
        out = torch.empty_like(y)
        comm.all_reduce(y, out, op="avg")
        stream.synchronize()
        return x.cpu(), out.cpu()

    res = run_emulated(world, fn)
    avg_ref = (sum(x.float() for x in xs) / world)
    for x, avg in res:
        # fp32 accumulation in rank order and one rounding: bit-exact against the reference
        assert torch.equal(x, ref)
        torch.testing.assert_close(avg.float(), avg_ref, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-2 if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("world", [2, 8])
def test_allreduce_ops_and_types(world):
    def fn(rank, world, comm, stream):
        out = {}
        a = (torch.arange(5000, dtype=torch.int32) * (rank + 3) % 1013).cuda()
        comm.all_reduce(a, op="max")
        out["max_i32"] = a.cpu()
        b = (torch.arange(3001, dtype=torch.int64) + rank).cuda()
        comm.all_reduce(b, op="sum")
        out["sum_i64"] = b.cpu()
        c = (torch.full((2049,), 1.0 + 0.01 * rank, dtype=torch.float64)).cuda()
        comm.all_reduce(c, op="prod")
        out["prod_f64"] = c.cpu()
        d = (torch.arange(777, dtype=torch.float16) - rank).cuda()
        comm.all_reduce(d, op="min")
        out["min_f16"] = d.cpu()
        stream.synchronize()
        return out

    res = run_emulated(world, fn)
    exp_max = torch.stack([torch.arange(5000, dtype=torch.int32) * (r + 3) % 1013 for r in range(world)]).max(0).values
    exp_sum = sum(torch.arange(3001, dtype=torch.int64) + r for r in range(world))
    exp_prod = torch.ones(2049, dtype=torch.float64)
    for r in range(world):
        exp_prod = exp_prod * (1.0 + 0.01 * r)
    exp_min = torch.arange(777, dtype=torch.float16) - (world - 1)
    for out in res:
        assert torch.equal(out["max_i32"], exp_max)
        assert torch.equal(out["sum_i64"], exp_sum)
        torch.testing.assert_close(out["prod_f64"], exp_prod)
        assert torch.equal(out["min_f16"], exp_min)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n", [1, 1000, 1 << 20])
def test_allgather_alltoall_broadcast_reduce(world, n):
    xs = _inputs(world, n, torch.bfloat16, seed=3)
    a2a = [torch.arange(world * n, dtype=torch.int32) + 1000003 * r for r in range(world)]

    def fn(rank, world, comm, stream):
        out = {}
        g = torch.empty(world * n, dtype=torch.bfloat16, device="cuda")
        comm.all_gather(xs[rank].cuda(), g)
        out["ag"] = g.cpu()
        # in-place all-gather
        g2 = torch.zeros(world * n, dtype=torch.bfloat16, device="cuda")
        g2[rank * n:(rank + 1) * n] = xs[rank].cuda()
        comm.all_gather(g2[rank * n:(rank + 1) * n], g2)
        out["ag_inplace"] = g2.cpu()
        t = torch.empty(world * n, dtype=torch.int32, device="cuda")
        comm.all_to_all(a2a[rank].cuda(), t)
        out["a2a"] = t.cpu()
        b = xs[rank].cuda()
        comm.broadcast(b, root=world - 1)
        out["bcast"] = b.cpu()
        r = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        comm.reduce(xs[rank].cuda(), r, root=1 % world)
        out["reduce"] = r.cpu()
        stream.synchronize()
        return out

    res = run_emulated(world, fn)
    exp_ag = torch.cat(xs)
    exp_red = _ordered_sum(xs, torch.bfloat16)
    for rank, out in enumerate(res):
        assert torch.equal(out["ag"], exp_ag)
        assert torch.equal(out["ag_inplace"], exp_ag)
        exp = torch.cat([a2a[j][rank * n:(rank + 1) * n] for j in range(world)])
        assert torch.equal(out["a2a"], exp)
        assert torch.equal(out["bcast"], xs[world - 1])
        if rank == 1 % world:
            assert torch.equal(out["reduce"], exp_red)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("n", [5, 4096 + 3, 1 << 19])
def test_reducescatter_and_fused_scale_cast(world, n):
    xs = _inputs(world, world * n, torch.float32, seed=5)

    def fn(rank, world, comm, stream):
        out = {}
        r = torch.empty(n, dtype=torch.float32, device="cuda")
        comm.reduce_scatter(xs[rank].cuda(), r)
        out["rs"] = r.cpu()
        # gradient averaging + fp32 -> bf16 cast in the same pass
        rb = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        comm.reduce_scatter(xs[rank].cuda(), rb, scale=1.0 / world)
        out["rs_bf16"] = rb.cpu()
        # bf16 gradients accumulated into fp32
        rf = torch.empty(n, dtype=torch.float32, device="cuda")
        comm.reduce_scatter(xs[rank].to(torch.bfloat16).cuda(), rf, scale=0.5)
        out["rs_up"] = rf.cpu()
        stream.synchronize()
        return out

    res = run_emulated(world, fn)
    for rank, out in enumerate(res):
        sl = slice(rank * n, (rank + 1) * n)
        acc = xs[0][sl].clone()
        for x in xs[1:]:
            acc = acc + x[sl]
        assert torch.equal(out["rs"], acc)
        assert torch.equal(out["rs_bf16"], (acc * (1.0 / world)).to(torch.bfloat16))
        accb = xs[0][sl].to(torch.bfloat16).float()
        for x in xs[1:]:
            accb = accb + x[sl].to(torch.bfloat16).float()
        assert torch.equal(out["rs_up"], accb * 0.5)


@pytest.mark.parametrize("world", [2, 4])
def test_sendrecv_ring_and_pairs(world):
    def fn(rank, world, comm, stream):
        from asystem_amem_b200 import group_end, group_start
        ok = True
        for n in (1, 4097, 1 << 20):
            s = torch.full((n,), float(rank + 1), device="cuda")
            r = torch.zeros(n, device="cuda")
            group_start()
            comm.send(s, (rank + 1) % world)
            comm.recv(r, (rank - 1) % world)
            group_end()
            stream.synchronize()
            ok = ok and bool((r == float((rank - 1) % world + 1)).all())
        return ok

    assert all(run_emulated(world, fn))


@pytest.mark.parametrize("world", [2, 4])
def test_all_to_all_v(world):
    cnt = lambda i, j: 0 if (i, j) == (0, 1) else (i + 2 * j + 1) * 1001  # noqa: E731

    def fn(rank, world, comm, stream):
        sc = [cnt(rank, j) for j in range(world)]
        rc = [cnt(j, rank) for j in range(world)]
        send = torch.cat([torch.full((sc[j],), 100.0 * rank + j, device="cuda", dtype=torch.bfloat16) for j in range(world)])
        recv = torch.full((sum(rc),), -1.0, device="cuda", dtype=torch.bfloat16)
        comm.all_to_all_v(send, recv, sc, rc)
        stream.synchronize()
        exp = torch.cat([torch.full((rc[j],), 100.0 * j + rank, dtype=torch.bfloat16) for j in range(world)])
        return torch.equal(recv.cpu(), exp)

    assert all(run_emulated(world, fn))


def test_unaligned_and_tiny_sizes():
    """Every size 1..130 elements and buffers at odd element offsets (no 16-byte alignment)."""
    world = 4
    base = _inputs(world, 4096, torch.float32, seed=9)

    def fn(rank, world, comm, stream):
        outs = []
        buf = base[rank].cuda()
        for n in list(range(1, 131)) + [1021]:
            x = buf[1:1 + n].clone()      # clone is aligned; use a view for the unaligned case
            y = buf[3:3 + n]              # 12-byte offset: not 16-byte aligned
            out = torch.empty(n + 1, device="cuda")[1:]
            comm.all_reduce(y, out)
            comm.all_reduce(x)
            outs.append((out.cpu(), x.cpu()))
        stream.synchronize()
        return outs

    res = run_emulated(world, fn)
    sizes = list(range(1, 131)) + [1021]
    for outs in res:
        for n, (o, x) in zip(sizes, outs):
            assert torch.equal(o, _ordered_sum([b[3:3 + n] for b in base], torch.float32))
            assert torch.equal(x, _ordered_sum([b[1:1 + n] for b in base], torch.float32))


@pytest.mark.parametrize("world,seed", [(2, 5), (4, 6)])
def test_random_cases_match_ordered_fp32_reference(world, seed):
    """Random (collective, type, size) cases on emulated ranks against a plain PyTorch fp32
    reference that adds in rank order and rounds once: results must be bit-identical.  Sizes go
    from one element to a few hundred thousand, so one-shot, two-shot, chunked and ragged-tail
    paths are all hit; the staging guard is checked at the end."""
    import random
    rnd = random.Random(seed)
    cases = []
    for c in range(40):
        kind = rnd.choice(["allreduce", "allgather", "reducescatter", "alltoall"])
        dtype = rnd.choice([torch.float32, torch.bfloat16, torch.float16])
        n = rnd.choice([1, 2, 3, 17, 255, 4097, 65537, rnd.randint(1, 300_000)])
        cases.append((c, kind, dtype, n))

    def data(r, n, dtype, salt):
        g = torch.Generator().manual_seed(1000 * salt + r)
        return torch.randn(n, generator=g).to(dtype)

    def ordered_sum(parts, dtype):
        acc = parts[0].float()
        for p in parts[1:]:
            acc = acc + p.float()
        return acc.to(dtype)

    def fn(rank, world, comm, stream):
        bad = []
        for c, kind, dtype, n in cases:
            if kind == "allreduce":
                xs = [data(r, n, dtype, c) for r in range(world)]
                x = xs[rank].cuda()
                comm.all_reduce(x)
                stream.synchronize()
                ok = torch.equal(x.cpu(), ordered_sum(xs, dtype))
            elif kind == "allgather":
                xs = [data(r, n, dtype, c) for r in range(world)]
                out = torch.empty(world * n, dtype=dtype, device="cuda")
                comm.all_gather(xs[rank].cuda(), out)
                stream.synchronize()
                ok = torch.equal(out.cpu(), torch.cat(xs))
            elif kind == "reducescatter":
                xs = [data(r, world * n, dtype, c) for r in range(world)]
                out = torch.empty(n, dtype=dtype, device="cuda")
                comm.reduce_scatter(xs[rank].cuda(), out)
                stream.synchronize()
                ok = torch.equal(out.cpu(), ordered_sum([x[rank * n:(rank + 1) * n] for x in xs], dtype))
            else:
                xs = [data(r, world * n, dtype, c) for r in range(world)]
                out = torch.empty(world * n, dtype=dtype, device="cuda")
                comm.all_to_all(xs[rank].cuda(), out)
                stream.synchronize()
                ok = torch.equal(out.cpu(), torch.cat([xs[j][rank * n:(rank + 1) * n] for j in range(world)]))
            if not ok:
                bad.append((c, kind, str(dtype), n))
        comm.check_canary()
        return bad

    for bad in run_emulated(world, fn):
        assert bad == [], bad
