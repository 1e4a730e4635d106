"""Hybrid layouts: carve a world communicator into tensor-parallel and expert/data-parallel
sub-communicators with ncclCommSplit.  All of them live in one process-wide registry, so
``pause_all()`` / ``resume_all()`` pause and resume them together (the reference pauses every
communicator of a process at once as well, whatever parallel layout created them).

Reference parity: the reference supports several communicators per process implicitly (its
registry is process-wide: nccl_patch/nccl_2.27.5-1.diff:70-77 ignores the comm argument,
README.md:259).
"""
from __future__ import annotations


def make_grid(world_comm, tp: int):
    """Returns (tp_comm, dp_comm): ranks [i*tp, (i+1)*tp) form a TP group, ranks with the same
    position inside their TP group form the EP/DP group."""
    if world_comm.nranks % tp:
        raise ValueError("world size must be a multiple of the tensor-parallel degree")
    r = world_comm.rank
    tp_comm = world_comm.split(r // tp, r)
    dp_comm = world_comm.split(r % tp, r)
    return tp_comm, dp_comm
