"""Expert-parallel MoE dispatch / combine on the fused kernels.

``MoeDispatcher`` owns the symmetric receive / expert-output buffers of one communicator.
``dispatch`` returns the rows of this rank's local experts already grouped by expert (the
routing permutation happens inside the all-to-all writes); ``combine`` pulls the expert outputs
back from the expert ranks and applies the routing weights in the same pass.
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
    send_pos: torch.Tensor        # int32 [T, k]: row of every (token, choice) on its expert's rank


class MoeDispatcher:
    def __init__(self, comm, num_experts: int, hidden: int, capacity_rows: int):
        if num_experts % comm.nranks:
            raise ValueError("experts must divide evenly over the ranks")
        self.comm, self.E, self.d, self.capacity = comm, num_experts, hidden, capacity_rows
        self.experts_per_rank = num_experts // comm.nranks
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
        T, k = topk_idx.shape
        counts = torch.empty(self.experts_per_rank, dtype=torch.int32, device=x.device)
        offsets = torch.empty(self.experts_per_rank + 1, dtype=torch.int32, device=x.device)
        send_pos = torch.empty(T, k, dtype=torch.int32, device=x.device)
        st = (stream or torch.cuda.current_stream()).cuda_stream
        B.check(self.comm.lib.amemMoeDispatch(x.data_ptr(), topk_idx.data_ptr(), T, k, self.d, self.E, self.capacity,
                                              counts.data_ptr(), offsets.data_ptr(), send_pos.data_ptr(), self.comm._h, st),
                "amemMoeDispatch")
        self._last_idx = topk_idx
        return DispatchResult(self.recv_x, counts, offsets, send_pos)

    def combine(self, topk_idx: torch.Tensor, topk_w: torch.Tensor, send_pos: torch.Tensor, out: torch.Tensor | None = None,
                stream=None) -> torch.Tensor:
        """Expert outputs must have been written to ``self.y`` in the row layout of ``recv_x``."""
        topk_idx = topk_idx.to(torch.int32).contiguous()
        topk_w = topk_w.to(torch.float32).contiguous()
        T, k = topk_idx.shape
        out = torch.empty(T, self.d, dtype=torch.bfloat16, device=topk_w.device) if out is None else out
        st = (stream or torch.cuda.current_stream()).cuda_stream
        B.check(self.comm.lib.amemMoeCombine(topk_idx.data_ptr(), topk_w.data_ptr(), send_pos.data_ptr(), out.data_ptr(), T, k,
                                             self.d, self.E, self.capacity, self.comm._h, st), "amemMoeCombine")
        return out
