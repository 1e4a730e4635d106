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


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m_local,N,K", [(128, 256, 256), (200, 520, 328), (512, 1024, 1024)])
def test_all_gather_gemm(world, m_local, N, K):
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
