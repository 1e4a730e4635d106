"""tcgen05 GEMM and its fused tensor-parallel forms against fp32 PyTorch references."""
import pytest
import torch

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


@pytest.fixture(params=["0", "1"], ids=["tiles128", "tiles256"])
def tile_height(request):
    """Forces the 128-row or the 256-row tile form of the plain GEMM (the library reads the
    variable at every call); without it the library picks by its cost model."""
    import os
    os.environ["AMEM_GEMM_TALL"] = request.param
    yield request.param
    os.environ.pop("AMEM_GEMM_TALL", None)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 1024), (1000, 264, 328), (4096, 4096, 4096), (77, 8, 8)])
def test_gemm_bf16_matches_fp32_reference(M, N, K, tile_height):
    from asystem_amem_b200.ops import gemm_bf16
    a, b = _rand((M, K), 1).cuda(), _rand((N, K), 2).cuda()
    out = gemm_bf16(a, b)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-2
    assert err <= tol, (err, tol)
    # bit-exact against the same product rounded once from fp32 where K is small enough for
    # the accumulation order not to matter
    if K <= 64:
        torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", [(256, 512, 4096), (1000, 264, 8192), (1000, 264, 2048), (4096, 4096, 4096), (8192, 3584, 8192), (520, 776, 4096)])
def test_gemm_split_k_tail(M, N, K, tile_height):
    """Shapes whose last wave of tiles is cut along K: partial accumulators meet in the
    workspace, the sum is taken in slice order, so repeated calls agree bit for bit, on the
    same stream and on a second one (which gets a workspace of its own)."""
    from asystem_amem_b200.ops import gemm_bf16
    a, b = _rand((M, K), 3).cuda(), _rand((N, K), 4, 0.05).cuda()
    outs = [gemm_bf16(a, b) for _ in range(3)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        outs.append(gemm_bf16(a, b))
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    tol = 2e-2 * ref.abs().max().item() + 1e-2
    for out in outs:
        assert (out.float() - ref).abs().max().item() <= tol
        assert torch.equal(out, outs[0])


_AG_VARIANTS = {   # AMEM_AG_DESIGN, AMEM_GEMM_TALL, AMEM_AG_MOVER, AMEM_AG_EPI_HELP
    "mover_warps_bulk_128": ("1", "0", "0", "0"),
    "mover_warps_bulk_256": ("1", "1", "0", "0"),
    "mover_warps_128": ("1", "0", "1", "0"),
    "mover_warps_256": ("1", "1", "1", "0"),
    "mover_warps_128_epilogue_helps": ("1", "0", "1", "1"),
    "mover_warps_256_epilogue_helps": ("1", "1", "1", "1"),
}


@pytest.fixture(params=list(_AG_VARIANTS), ids=list(_AG_VARIANTS))
def ag_variant(request):
    """The mover-warp schedule of the all-gather -> GEMM kernel at every rank count: both tile
    heights, both ways of copying, with and without help from the epilogue warps (the schedule
    with dedicated mover CTAs has a test file of its own).  The library reads the variables at
    every call."""
    import os
    names = ("AMEM_AG_DESIGN", "AMEM_GEMM_TALL", "AMEM_AG_MOVER", "AMEM_AG_EPI_HELP")
    for name, val in zip(names, _AG_VARIANTS[request.param]):
        os.environ[name] = val
    yield request.param
    for name in names:
        os.environ.pop(name, None)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m_local,N,K", [(128, 256, 256), (200, 520, 328), (512, 1024, 1024), (300, 264, 4096)])
def test_all_gather_gemm(world, m_local, N, K, ag_variant):
    """Both tile heights; shards whose row count is no multiple of the tile height or of the rows
    one ready flag covers (a flag covers 16 rows at K = 256, 13 at K = 328, one at K = 4096)."""
    from asystem_amem_b200.ops import all_gather_gemm
    shards = [_rand((m_local, K), 10 + r) for r in range(world)]
    weights = [_rand((N, K), 50 + r, 0.05) for r in range(world)]
    full = torch.cat(shards).float()

    def fn(rank, world, comm, stream):
        outs = []
        for _ in range(2):   # second call reuses the gathered buffer (cross-launch guard)
            outs.append(all_gather_gemm(comm, shards[rank].cuda(), weights[rank].cuda()).cpu())
        return outs

    res = run_emulated(world, fn)
    for rank, outs in enumerate(res):
        ref = full @ weights[rank].float().t()
        tol = 2e-2 * ref.abs().max().item() + 1e-2
        for out in outs:
            assert (out.float() - ref).abs().max().item() <= tol
        assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m_local,N,K", [(128, 256, 256), (136, 264, 200), (256, 1024, 512)])
def test_gemm_reduce_scatter(world, m_local, N, K):
    from asystem_amem_b200.ops import gemm_reduce_scatter
    M = m_local * world
    acts = [_rand((M, K), 20 + r) for r in range(world)]
    weights = [_rand((N, K), 70 + r, 0.05) for r in range(world)]

    def fn(rank, world, comm, stream):
        outs = []
        for _ in range(2):
            outs.append(gemm_reduce_scatter(comm, acts[rank].cuda(), weights[rank].cuda()).cpu())
        return outs

    res = run_emulated(world, fn)
    # reference: every rank's partial rounded to bf16 (as it travels), summed in fp32 in rank order
    parts = [(acts[r].float() @ weights[r].float().t()) for r in range(world)]
    for rank, outs in enumerate(res):
        sl = slice(rank * m_local, (rank + 1) * m_local)
        exact = sum(p[sl] for p in parts)
        tol = 3e-2 * exact.abs().max().item() + 2e-2
        for out in outs:
            assert (out.float() - exact).abs().max().item() <= tol
        assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("counts,N,K", [([128, 256], 256, 64), ([5, 0, 300, 1, 129, 77], 264, 328), ([1000, 3, 0, 0, 2000, 511, 640, 130], 3072, 512),
                                          ([0, 0, 0], 128, 64)])
def test_grouped_gemm_reads_device_offsets(counts, N, K):
    """One launch multiplies every group's rows by that group's matrix; groups start at rows of any
    alignment, some are empty, the offsets never leave the device, rows past the last group stay
    as they were."""
    from asystem_amem_b200.ops import grouped_gemm_bf16
    groups, total = len(counts), sum(counts)
    cap = total + 200
    a = _rand((cap, K), 5).cuda()
    w = _rand((groups, N, K), 6, 0.05).cuda()
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32).cuda()
    out = torch.full((cap, N), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm_bf16(a, w, offs, out=out, rows_hint=total)
    again = torch.full((cap, N), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm_bf16(a, w, offs, out=again)
    torch.cuda.synchronize()
    lo = 0
    for e, c in enumerate(counts):
        ref = a[lo:lo + c].float() @ w[e].float().t()
        if c:
            err = (out[lo:lo + c].float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-2, (e, err)
        lo += c
    assert bool((out[total:] == 7.0).all())          # nothing stored outside the groups
    assert torch.equal(out, again)


@pytest.mark.parametrize("counts,ffn,K", [([200, 0, 57], 64, 128), ([300, 129, 1, 640], 1536, 512)])
def test_grouped_gemm_swiglu_epilogue(counts, ffn, K):
    """gate / up projection with silu(gate) * up computed in the epilogue on the fp32 accumulators."""
    from asystem_amem_b200.ops import grouped_gemm_bf16, interleave_gate_up
    groups, total = len(counts), sum(counts)
    a = _rand((total + 10, K), 8).cuda()
    w13 = _rand((groups, 2 * ffn, K), 9, 0.05).cuda()
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32).cuda()
    out = grouped_gemm_bf16(a, interleave_gate_up(w13, ffn), offs, rows_hint=total, swiglu=True)
    torch.cuda.synchronize()
    assert out.shape == (total + 10, ffn)
    lo = 0
    for e, c in enumerate(counts):
        h = a[lo:lo + c].float() @ w13[e].float().t()
        ref = torch.nn.functional.silu(h[:, :ffn]) * h[:, ffn:]
        if c:
            err = (out[lo:lo + c].float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-2, (e, err)
        lo += c


def test_grouped_linear_gradients():
    """GroupedLinear (forward and input gradient on the grouped kernel, weight gradient per group)
    against autograd on a per-group loop in fp32."""
    from asystem_amem_b200.models.moe_layer import GroupedLinear
    counts, N, K = [130, 0, 77, 300], 192, 256
    groups, total = len(counts), sum(counts)
    rows = _rand((total, K), 11).cuda().requires_grad_(True)
    w = _rand((groups, N, K), 12, 0.05).cuda().requires_grad_(True)
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32).cuda()
    gout = _rand((total, N), 13).cuda()
    out = GroupedLinear.apply(rows, w, offs)
    out.backward(gout)
    torch.cuda.synchronize()
    r32 = rows.detach().float().requires_grad_(True)
    w32 = w.detach().float().requires_grad_(True)
    lo = 0
    pieces = []
    for e, c in enumerate(counts):
        pieces.append(r32[lo:lo + c] @ w32[e].t())
        lo += c
    ref = torch.cat(pieces)
    ref.backward(gout.float())
    scale = lambda t: 2e-2 * t.abs().max().item() + 2e-2  # noqa: E731
    assert (out.float() - ref).abs().max().item() <= scale(ref)
    assert (rows.grad.float() - r32.grad).abs().max().item() <= scale(r32.grad)
    assert (w.grad.float() - w32.grad).abs().max().item() <= scale(w32.grad)
