"""All-gather -> GEMM on the schedule with dedicated mover CTAs (what a communicator of five or
more ranks runs; forced here for two and four ranks too) against an fp32 PyTorch reference."""
import os

import pytest
import torch

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


@pytest.fixture
def mover_ctas():
    os.environ["AMEM_AG_DESIGN"] = "2"
    yield
    os.environ.pop("AMEM_AG_DESIGN", None)


def _check(world, m_local, N, K):
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
@pytest.mark.parametrize("m_local,N,K", [(128, 256, 256), (200, 520, 328), (512, 1024, 1024), (300, 264, 4096)])
def test_all_gather_gemm_with_mover_ctas(world, m_local, N, K, mover_ctas):
    _check(world, m_local, N, K)


@pytest.mark.parametrize("m_local,N,K", [(128, 256, 256), (512, 1024, 1024)])
def test_eight_ranks_pick_the_mover_cta_schedule_by_themselves(m_local, N, K):
    """No variable set: eight ranks run the mover-CTA schedule (amemAllGatherGemmPlan says so) and
    the result is right."""
    import ctypes
    from asystem_amem_b200.bindings import load_library
    os.environ.pop("AMEM_AG_DESIGN", None)
    warps = ctypes.c_int(-1)
    assert load_library().amemAllGatherGemmPlan(8, m_local, K, ctypes.byref(warps), None, None) == 0 and warps.value == 0
    _check(8, m_local, N, K)
