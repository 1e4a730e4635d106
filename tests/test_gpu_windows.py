"""Registered windows on the GPU (ranks emulated on cuda:0, so the peer-load / peer-store form of
the in-place all-reduce runs; the multicast form needs one GPU per rank and is covered by
tests/test_gpu_multiproc.py when several GPUs are present)."""
import pytest
import torch

from gpu_util import run_emulated

pytestmark = pytest.mark.gpu


def _ordered_sum(xs, dtype):
    ref = xs[0].float()
    for x in xs[1:]:
        ref = ref + x.float()
    return ref.to(dtype)


@pytest.mark.parametrize("world,dtype,n", [(2, torch.bfloat16, 1 << 20), (4, torch.float32, 300_001), (8, torch.bfloat16, 777_777)])
def test_window_allreduce_in_place_matches_ordered_fp32_sum(world, dtype, n):
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, generator=g).to(dtype) for _ in range(world)]
    es = xs[0].element_size()

    def fn(rank, world, comm, stream):
        win = comm.window_alloc(n * es + 4096)
        x = win.tensor(dtype, n)
        x.copy_(xs[rank])
        stream.synchronize()
        comm.all_reduce(x, algo="window")
        stream.synchronize()
        first = x.clone()
        tail = win.tensor(torch.uint8, 4096, offset_bytes=n * es)
        tail.fill_(rank + 3)
        same = True
        for cycle in range(3):
            f0 = torch.cuda.mem_get_info()[0]
            comm.pause()
            freed = torch.cuda.mem_get_info()[0] - f0
            comm.resume()
            same = same and torch.equal(x, first) and bool((tail == rank + 3).all())   # contents came back
            x.copy_(xs[rank])
            stream.synchronize()
            comm.all_reduce(x)                      # picked by the tuner
            stream.synchronize()
            same = same and torch.equal(x, first)
        out = first.cpu()
        win.free()
        return same, out, freed

    res = run_emulated(world, fn)
    ref = _ordered_sum(xs, dtype)
    for same, first, freed in res:
        assert same
        assert torch.equal(first, ref)


def test_window_out_of_place_and_small_sizes():
    world = 4
    g = torch.Generator().manual_seed(9)
    sizes = [1, 7, 130, 4097, 70_001]
    xs = [torch.randn(max(sizes), generator=g) for _ in range(world)]

    def fn(rank, world, comm, stream):
        a = comm.window_alloc(4 << 20)
        b = comm.window_alloc(4 << 20)
        ok = True
        for i, n in enumerate(sizes):
            off = 4 * (3 * i)                        # odd element offsets: the unaligned path
            src = a.tensor(torch.float32, n, offset_bytes=off)
            dst = b.tensor(torch.float32, n, offset_bytes=off)
            src.copy_(xs[rank][:n])
            dst.zero_()
            stream.synchronize()
            comm.all_reduce(src, dst, algo="window")
            stream.synchronize()
            ref = _ordered_sum([x[:n].cuda() for x in xs], torch.float32)
            ok = ok and torch.equal(dst, ref) and torch.equal(src, xs[rank][:n].cuda())
        b.free()
        a.free()
        return ok

    assert all(run_emulated(world, fn))
