"""amemMoePermuteNoAlloc, the routing permutation that allocates nothing, against the regular
dispatch entry point.

Some callers cannot get device memory when they need to group tokens by expert: their
communicators are paused (no receive buffers exist and tracked allocations are refused), or
they share the GPU and their budget is fully handed out.  For them the library offers one
entry point whose scratch lives in a fixed device array inside the library.  Here it is called
through its exported C symbol, twice in a row with different shapes (the array keeps the first
call's contents), and compared bit for bit with amemMoeDispatch on a one-rank communicator.
This file is collected last so that a failure here cannot hide the other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(comm, x, idx, E, cap):
    from asystem_amem_b200.ops import MoeDispatcher
    disp = MoeDispatcher(comm, E, x.shape[1], cap)
    res = disp.dispatch(x, idx)
    torch.cuda.synchronize()
    total = int(res.expert_offsets[-1])
    return res.recv_x[:total].clone(), res.expert_counts.clone(), res.expert_offsets.clone(), res.send_pos.clone()


def _no_alloc(lib, x, idx, E, cap):
    T, k = idx.shape
    d = x.shape[1]
    recv = torch.zeros(cap, d, dtype=torch.bfloat16, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    offs = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    pos = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.amemMoePermuteNoAlloc(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(idx.data_ptr()), T, k, d, E,
                                   ctypes.c_void_p(recv.data_ptr()), cap, ctypes.c_void_p(counts.data_ptr()),
                                   ctypes.c_void_p(offs.data_ptr()), ctypes.c_void_p(pos.data_ptr()),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.amemLastError()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    total = int(offs[-1])
    return recv[:total], counts, offs, pos, free_before - torch.cuda.mem_get_info()[0]


def _torch_oracle(x, idx, E, cap):
    """The permutation written out in plain torch: rows grouped by expert, (token, choice) order
    inside an expert; what does not fit in `cap` rows is left out."""
    T, k = idx.shape
    flat = idx.reshape(-1).long().cpu()
    order = torch.argsort(flat, stable=True)
    pos = torch.empty_like(flat)
    pos[order] = torch.arange(flat.numel())
    kept = order[:cap]
    rows = x.cpu()[kept // k]
    counts = torch.bincount(flat[kept], minlength=E).to(torch.int32)
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(counts, 0)
    pos = torch.where(pos < cap, pos, torch.full_like(pos, -1)).to(torch.int32).view(T, k)
    return rows, counts, offs, pos


def test_no_alloc_permute_matches_dispatch_twice():
    from asystem_amem_b200 import Communicator, get_unique_id, load_library
    lib = load_library()
    lib.amemMoePermuteNoAlloc.restype = ctypes.c_int
    torch.cuda.set_device(0)
    comm = Communicator(1, 0, get_unique_id())
    g = torch.Generator().manual_seed(42)
    took = []
    for (T, k, d, E) in [(777, 4, 256, 64), (300, 8, 128, 256)]:
        x = torch.randn(T, d, generator=g).to(torch.bfloat16).cuda()
        idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
        cap = T * k
        ref = _reference(comm, x, idx, E, cap)
        got = _no_alloc(lib, x, idx, E, cap)
        for a, b in zip(ref, got[:4]):
            assert torch.equal(a, b)
        for a, b in zip(_torch_oracle(x, idx, E, cap), got[:4]):    # and against plain torch
            assert torch.equal(a, b.cpu())
        took.append(got[4])
        # a buffer that is too small: the tail is left out, the offsets stay inside the buffer
        small = cap // 2 + 3
        got = _no_alloc(lib, x, idx, E, small)
        for a, b in zip(_torch_oracle(x, idx, E, small), got[:4]):
            assert torch.equal(a, b.cpu())
        assert int(got[2][-1]) == small and int((got[3] < 0).sum()) == cap - small
    # the second call found the library already set up: the device's free memory did not move
    assert took[1] <= 0
    # sizes beyond the built-in scratch are refused with a message, nothing is launched
    rc = lib.amemMoePermuteNoAlloc(None, None, 8, 1, 8, 257, None, 8, None, None, None, None)
    assert rc == 4 and b"at most 256" in lib.amemLastError()
    comm.destroy()
