"""Pause / resume on the GPU: memory really returns to the driver (cudaMemGetInfo), addresses
and control state survive, results stay bit-identical over many cycles, collectives are refused
while paused.  Ranks are emulated on cuda:0."""
import ctypes

import pytest
import torch

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


def test_single_rank_pause_frees_memory_and_keeps_user_data(monkeypatch):
    from asystem_amem_b200 import Communicator, NcclError, get_unique_id, mem_alloc, mem_free, mem_stats, pause_all, resume_all
    torch.cuda.set_device(0)
    monkeypatch.setenv("AMEM_PAUSE_CONTROL", "1")     # release the control segment as well
    comm = Communicator(1, 0, get_unique_id())
    stage = comm.info()["stage_bytes"]
    nbytes = 64 << 20
    p = mem_alloc(nbytes)
    # view the VMM allocation as a tensor through the CUDA array interface
    class Holder:
        __cuda_array_interface__ = {"shape": (nbytes // 4,), "typestr": "<f4", "data": (p, False), "version": 3}
    t = torch.as_tensor(Holder(), device="cuda")
    ref = torch.randn(nbytes // 4, device="cuda")
    t.copy_(ref)
    x = torch.randn(1 << 20, device="cuda")
    y = torch.empty_like(x)
    comm.all_reduce(x, y)
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    free0, _ = torch.cuda.mem_get_info()
    pause_all()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 - free0 >= stage + nbytes, (free0, free1, stage)
    with pytest.raises(NcclError) as ei:
        comm.all_reduce(x, y)
    assert ei.value.code == 5
    st = mem_stats()
    assert st["paused"] == 1 and st["live_bytes"] <= (2 << 20)   # at most the plain GEMM's resident protocol words, if a GEMM ran in this process
    resume_all()
    free2, _ = torch.cuda.mem_get_info()
    assert abs(free2 - free0) <= (4 << 20)
    assert torch.equal(t, ref)          # same address, same contents
    comm.all_reduce(x, y)
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    ps = comm.pause_resume_stats()
    assert ps["bytes_offloaded"] < ps["bytes_released_local"]   # staging was dropped, not copied
    del t
    mem_free(p)
    comm.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_emulated_ranks_cycles_bitwise(world):
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(1 << 18, generator=g).to(torch.bfloat16) for _ in range(world)]

    def fn(rank, world, comm, stream):
        x = xs[rank].cuda()
        first = torch.empty_like(x)
        comm.all_reduce(x, first)
        gathered = torch.empty(world * 1000, dtype=torch.bfloat16, device="cuda")
        comm.all_gather(x[:1000], gathered)
        stream.synchronize()
        frees = []
        same = True
        for cycle in range(6):
            f0, _ = torch.cuda.mem_get_info()
            comm.pause()
            comm.pause()                    # idempotent
            frees.append(torch.cuda.mem_get_info()[0] - f0)
            comm.resume()
            out = torch.empty_like(x)
            comm.all_reduce(x, out)
            g2 = torch.empty_like(gathered)
            comm.all_gather(x[:1000], g2)
            stream.synchronize()
            same = same and torch.equal(out, first) and torch.equal(g2, gathered)
        return same, frees, first.cpu()

    res = run_emulated(world, fn)
    ref = xs[0].float()
    for x in xs[1:]:
        ref = ref + x.float()
    ref = ref.to(torch.bfloat16)
    for same, frees, first in res:
        assert same
        assert torch.equal(first, ref)


def test_process_wide_pause_with_emulated_ranks():
    """ncclPause(NULL) from one thread while the process holds all ranks of a communicator."""
    import threading
    from asystem_amem_b200 import pause_all, resume_all, mem_stats
    world = 4
    barrier = threading.Barrier(world)

    def fn(rank, world, comm, stream):
        x = torch.full((4096,), float(rank + 1), device="cuda")
        comm.all_reduce(x)
        stream.synchronize()
        barrier.wait()
        freed = None
        if rank == 0:
            f0, _ = torch.cuda.mem_get_info()
            pause_all()
            freed = torch.cuda.mem_get_info()[0] - f0
            live = mem_stats()["live_bytes"]    # only resident blocks: the ranks' control segments (and the plain GEMM's, if one ran)
            assert world * world * (2 << 20) <= live <= world * world * (2 << 20) + (4 << 20)
            resume_all()
        barrier.wait()
        y = torch.full((4096,), float(rank + 1), device="cuda")
        comm.all_reduce(y)
        stream.synchronize()
        return bool((y == x).all()), freed

    res = run_emulated(world, fn)
    assert all(r[0] for r in res)
    stage_total = res[0][1]
    assert stage_total is not None and stage_total > (world * 200 << 20)


def test_work_memory_of_the_fused_kernels_is_tracked_and_returned():
    """The split-K workspace of the plain GEMM and the MoE work area are tracked allocations:
    ncclMemStats accounts for them, ncclPause(NULL) returns them, and the kernels work again after
    ncclResume (the GEMM also runs while paused, without its workspace)."""
    from asystem_amem_b200 import Communicator, get_unique_id, mem_stats, pause_all, resume_all
    from asystem_amem_b200.ops import MoeDispatcher, gemm_bf16
    torch.cuda.set_device(0)
    comm = Communicator(1, 0, get_unique_id())
    a = torch.randn(1000, 4096, device="cuda").to(torch.bfloat16)
    b = (torch.randn(264, 4096, device="cuda") * 0.05).to(torch.bfloat16)
    ref = gemm_bf16(a, b)                                   # a shape whose last wave is split along K
    disp = MoeDispatcher(comm, 8, 64, 256)
    idx = torch.randint(0, 8, (64, 2), device="cuda", dtype=torch.int32)
    x = torch.randn(64, 64, device="cuda").to(torch.bfloat16)
    res = disp.dispatch(x, idx)
    torch.cuda.synchronize()
    first_pos = res.send_pos.clone()
    mid = mem_stats()
    # everything mapped now: staging + control, the split-K workspace (about 28 MB; an earlier test of
    # this process may have made it already) + its counters, the MoE buffers and work area
    assert mid["live_bytes"] >= comm.info()["stage_bytes"] + (24 << 20), mid
    f0 = torch.cuda.mem_get_info()[0]
    pause_all()
    freed = torch.cuda.mem_get_info()[0] - f0
    assert freed >= mid["live_bytes"] - (8 << 20), (freed, mid)    # all but the small resident blocks came back
    while_paused = gemm_bf16(a, b)                          # no workspace now: same product, unsplit
    torch.cuda.synchronize()
    resume_all()
    again = gemm_bf16(a, b)
    res2 = disp.dispatch(x, idx)
    torch.cuda.synchronize()
    full = a.float() @ b.float().t()
    tol = 2e-2 * full.abs().max().item() + 1e-2
    assert (while_paused.float() - full).abs().max().item() <= tol
    assert torch.equal(again, ref) and torch.equal(res2.send_pos, first_pos)
    comm.destroy()
