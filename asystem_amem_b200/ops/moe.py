"""Expert-parallel MoE dispatch / combine on the fused kernels.

``MoeDispatcher`` owns the symmetric receive / expert-output buffers of one communicator.
``dispatch`` returns the rows of this rank's local experts already grouped by expert (the
routing permutation happens inside the all-to-all writes); ``combine`` pulls the expert outputs
back from the expert ranks and applies the routing weights in the same pass.

On the mock backend (no GPU) the dispatcher composes the same row layout from the library's
all-gather and variable-size all-to-all on host tensors, which is how the expert-parallel
wrappers and their gradients are tested as multi-process runs on a CPU.  CUDA tensors always
go to the kernels.

Reference parity: none -- the reference names all-to-all as the largest consumer of NCCL memory
(README.md:132) but leaves routing and permutation to the framework above it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import bindings as B


def _view(ptr: int, rows: int, d: int, device) -> torch.Tensor:
    """A bf16 [rows, d] tensor over library-owned device memory (no ownership transfer)."""
    class _Holder:
        __cuda_array_interface__ = {"shape": (rows * d,), "typestr": "<i2", "data": (ptr, False), "version": 3}
    return torch.as_tensor(_Holder(), device=device).view(torch.bfloat16).view(rows, d)


@dataclass
class DispatchResult:
    recv_x: torch.Tensor          # bf16 [capacity_rows, d]; rows [0, total_rows) are valid
    expert_counts: torch.Tensor   # int32 [experts_per_rank]
    expert_offsets: torch.Tensor  # int32 [experts_per_rank + 1]
    send_pos: torch.Tensor        # int32 [T, k]: row of every (token, choice) on its expert's rank (-1: left out, no room)
    dropped: torch.Tensor | None = None   # int32 [1]: rows routed to THIS rank that did not fit its capacity


class MoeDispatcher:
    def __init__(self, comm, num_experts: int, hidden: int, capacity_rows: int):
        if num_experts % comm.nranks:
            raise ValueError("experts must divide evenly over the ranks")
        self.comm, self.E, self.d, self.capacity = comm, num_experts, hidden, capacity_rows
        self.experts_per_rank = num_experts // comm.nranks
        from ..comm import backend_usage
        self.host = backend_usage()["backend"] == "mock"   # no GPU: composed from all_gather + all_to_all_v
        if self.host:
            self.device = torch.device("cpu")
            self.recv_x = torch.zeros(capacity_rows, hidden, dtype=torch.bfloat16)
            self.y = torch.zeros(capacity_rows, hidden, dtype=torch.bfloat16)
            return
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._map_buffers()

    def _map_buffers(self) -> None:
        rx, y = ctypes.c_void_p(), ctypes.c_void_p()
        B.check(self.comm.lib.amemMoeBuffers(self.comm._h, self.capacity, self.d, ctypes.byref(rx), ctypes.byref(y)), "amemMoeBuffers")
        self.recv_x = _view(rx.value, self.capacity, self.d, self.device)
        self.y = _view(y.value, self.capacity, self.d, self.device)  # experts write their outputs here

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, stream=None) -> DispatchResult:
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == self.d
        topk_idx = topk_idx.to(torch.int32).contiguous()
        if self.host:
            return self._host_dispatch(x, topk_idx)
        T, k = topk_idx.shape
        counts = torch.empty(self.experts_per_rank, dtype=torch.int32, device=x.device)
        offsets = torch.empty(self.experts_per_rank + 1, dtype=torch.int32, device=x.device)
        send_pos = torch.empty(T, k, dtype=torch.int32, device=x.device)
        dropped = torch.zeros(1, dtype=torch.int32, device=x.device)
        st = (stream or torch.cuda.current_stream()).cuda_stream
        B.check(self.comm.lib.amemMoeDispatchCounted(x.data_ptr(), topk_idx.data_ptr(), T, k, self.d, self.E, self.capacity,
                                                     counts.data_ptr(), offsets.data_ptr(), send_pos.data_ptr(), dropped.data_ptr(),
                                                     self.comm._h, st), "amemMoeDispatch")
        self._last_idx = topk_idx
        return DispatchResult(self.recv_x, counts, offsets, send_pos, dropped)

    def combine(self, topk_idx: torch.Tensor, topk_w: torch.Tensor, send_pos: torch.Tensor, out: torch.Tensor | None = None,
                stream=None) -> torch.Tensor:
        """Expert outputs must have been written to ``self.y`` in the row layout of ``recv_x``."""
        topk_idx = topk_idx.to(torch.int32).contiguous()
        topk_w = topk_w.to(torch.float32).contiguous()
        if self.host:
            res = self._host_combine(topk_idx, topk_w, send_pos)
            return res if out is None else out.copy_(res)
        T, k = topk_idx.shape
        out = torch.empty(T, self.d, dtype=torch.bfloat16, device=topk_w.device) if out is None else out
        st = (stream or torch.cuda.current_stream()).cuda_stream
        B.check(self.comm.lib.amemMoeCombine(topk_idx.data_ptr(), topk_w.data_ptr(), send_pos.data_ptr(), out.data_ptr(), T, k,
                                             self.d, self.E, self.capacity, self.comm._h, st), "amemMoeCombine")
        return out

    # ---- host form (mock backend): same row layout as the kernels, built from the library's
    # all-gather and variable-size all-to-all, so that the expert-parallel wrappers and their
    # gradients can be tested as real multi-process runs without a GPU ------------------------
    def _host_plan(self, topk_idx: torch.Tensor):
        """Everything both directions need, from the routing alone (every rank computes the same
        global picture): sorted pair order, destination rows, per-peer element counts."""
        n, me, El = self.comm.nranks, self.comm.rank, self.experts_per_rank
        flat = topk_idx.reshape(-1).long()                              # pair p = t * k + c
        cnt = torch.bincount(flat, minlength=self.E)                    # my pairs per expert
        all_cnt = torch.empty(n, self.E, dtype=torch.int64)
        self.comm.all_gather(cnt.contiguous(), all_cnt)                 # all_cnt[src][e]
        total = all_cnt.sum(0)
        exp_off = torch.zeros(self.E, dtype=torch.int64)                # first row of expert e at its owner
        for r in range(n):
            seg = total[r * El:(r + 1) * El]
            exp_off[r * El:(r + 1) * El] = torch.cumsum(seg, 0) - seg
        src_off = torch.cumsum(all_cnt, 0) - all_cnt                    # rows of expert e from lower source ranks
        order = torch.argsort(flat, stable=True)                        # pairs by expert, pair order inside
        starts = torch.cumsum(cnt, 0) - cnt
        within = torch.empty_like(flat)
        within[order] = torch.arange(flat.numel()) - starts[flat[order]]
        pos = exp_off[flat] + src_off[me][flat] + within
        pos = torch.where(pos < self.capacity, pos, torch.full_like(pos, -1))
        send_rows = torch.tensor([int(cnt[r * El:(r + 1) * El].sum()) for r in range(n)])
        recv_rows = torch.tensor([int(all_cnt[r][me * El:(me + 1) * El].sum()) for r in range(n)])
        return flat, order, pos, all_cnt, total, send_rows, recv_rows

    def _owner_permutation(self, all_cnt: torch.Tensor) -> torch.Tensor:
        """Rows arrive grouped [source][local expert]; the buffers hold them [local expert][source]:
        returns, for every row in arrival order, its row in the buffer."""
        n, me, El = self.comm.nranks, self.comm.rank, self.experts_per_rank
        mine = all_cnt[:, me * El:(me + 1) * El]                         # [src][el]
        per_el = mine.sum(0)
        el_off = torch.cumsum(per_el, 0) - per_el
        src_in_el = torch.cumsum(mine, 0) - mine                        # [src][el] offset inside the expert
        rows = []
        for src in range(n):
            for el in range(El):
                c = int(mine[src][el])
                rows.append(torch.arange(c) + int(el_off[el]) + int(src_in_el[src][el]))
        return torch.cat(rows) if rows else torch.zeros(0, dtype=torch.int64)

    def _host_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor) -> DispatchResult:
        T, k = topk_idx.shape
        me, El, d = self.comm.rank, self.experts_per_rank, self.d
        flat, order, pos, all_cnt, total, send_rows, recv_rows = self._host_plan(topk_idx)
        if int((pos < 0).sum()):
            raise ValueError("host form of the MoE dispatch needs a capacity that holds every routed row")
        send = x[order // k].contiguous()
        arrive = torch.empty(int(recv_rows.sum()), d, dtype=x.dtype)
        self.comm.all_to_all_v(send.view(-1), arrive.view(-1), (send_rows * d).tolist(), (recv_rows * d).tolist())
        self.recv_x[self._owner_permutation(all_cnt)] = arrive
        counts = total[me * El:(me + 1) * El].to(torch.int32)
        offsets = torch.zeros(El + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(counts, 0)
        return DispatchResult(self.recv_x, counts, offsets, pos.to(torch.int32).view(T, k))

    def _host_combine(self, topk_idx: torch.Tensor, topk_w: torch.Tensor, send_pos: torch.Tensor) -> torch.Tensor:
        T, k = topk_idx.shape
        d = self.d
        flat, order, _pos, all_cnt, _total, send_rows, recv_rows = self._host_plan(topk_idx)
        back = self.y[self._owner_permutation(all_cnt)].contiguous()     # arrival order = what each source sent
        got = torch.empty(int(send_rows.sum()), d, dtype=self.y.dtype)
        self.comm.all_to_all_v(back.view(-1), got.view(-1), (recv_rows * d).tolist(), (send_rows * d).tolist())
        y_at = torch.empty(T * k, d, dtype=self.y.dtype)
        y_at[order] = got                                                # rows came back in sorted pair order
        out = (y_at.view(T, k, d).float() * topk_w.view(T, k, 1)).sum(1)
        return out.to(torch.bfloat16)
