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
