"""High-level communicator over the native library.

One :class:`Communicator` per rank.  Collectives take torch tensors (CUDA tensors with the
CUDA backend; CPU tensors with ``AMEM_BACKEND=mock``) or numpy arrays and run on the current
torch CUDA stream unless ``stream`` is given.  ``pause()`` / ``resume()`` release and restore
the communicator's device memory; :func:`pause_all` / :func:`resume_all` do so for every
communicator of the process (the reference's ``ncclPause(NULL)`` / ``ncclResume(NULL)``).

Reference parity: the pynccl-style integration the reference documents for SGLang / vLLM
(README.md:262-294: load the patched libnccl, call ncclPause / ncclResume / ncclSetGroupID
through ctypes); here the same calls plus the collectives sit behind one Communicator class.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Optional

from . import bindings as B


def _torch():
    import torch
    return torch


def _dtype_code(t) -> int:
    name = str(t.dtype).replace("torch.", "")
    if name not in B.DTYPES:
        raise TypeError(f"unsupported dtype {t.dtype}")
    return B.DTYPES[name]


def _ptr(t) -> int:
    if hasattr(t, "data_ptr"):
        if not t.is_contiguous():
            raise ValueError("collectives need contiguous tensors")
        return t.data_ptr()
    return t.ctypes.data  # numpy


def _numel(t) -> int:
    return t.numel() if hasattr(t, "numel") else t.size


def _stream_handle(stream, tensor) -> int:
    if stream is not None:
        return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
    if hasattr(tensor, "is_cuda") and tensor.is_cuda:
        return _torch().cuda.current_stream(tensor.device).cuda_stream
    return 0


def get_unique_id() -> bytes:
    lib = B.load_library()
    uid = B.UniqueId()
    B.check(lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
    return bytes(uid)


def set_group_id(group_id: int) -> None:
    B.check(B.load_library().ncclSetGroupID(group_id), "ncclSetGroupID")


def get_group_id() -> int:
    v = ctypes.c_int()
    B.check(B.load_library().ncclGetGroupID(ctypes.byref(v)), "ncclGetGroupID")
    return v.value


def mem_stats(print_too: bool = False) -> dict:
    lib = B.load_library()
    if print_too:
        lib.ncclMemStats()
    s = B.MemStats()
    B.check(lib.amemMemStatsGet(ctypes.byref(s)), "amemMemStatsGet")
    return B.struct_to_dict(s)


def backend_usage() -> dict:
    lib = B.load_library()
    phys, maps, name = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_char_p()
    B.check(lib.amemBackendUsage(ctypes.byref(phys), ctypes.byref(maps), ctypes.byref(name)), "amemBackendUsage")
    return {"physical_bytes": phys.value, "mappings": maps.value, "backend": name.value.decode()}


def backend_timings(reset: bool = False) -> dict:
    """Wall time and call count of every kind of VMM driver call made so far."""
    import json
    buf = ctypes.create_string_buffer(2048)
    lib = B.load_library()
    lib.amemBackendTimings.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int]
    B.check(lib.amemBackendTimings(buf, 2048, 1 if reset else 0), "amemBackendTimings")
    return json.loads(buf.value.decode() or "{}")


def pause_all() -> None:
    B.check(B.load_library().ncclPause(None), "ncclPause")


def resume_all() -> None:
    B.check(B.load_library().ncclResume(None), "ncclResume")


@contextlib.contextmanager
def paused(*comms):
    """``with paused():`` hands every communicator (and ncclMemAlloc buffer) of the process back
    to the driver for the duration of the block; ``with paused(a, b):`` only the named
    communicators.  Everything is resumed on the way out, also when the block raises.  Every rank
    must enter and leave the block, like ncclPause / ncclResume themselves."""
    if comms:
        for c in comms:
            c.pause()
    else:
        pause_all()
    try:
        yield
    finally:
        if comms:
            for c in comms:
                c.resume()
        else:
            resume_all()


def process_pause_resume_stats() -> dict:
    s = B.PauseResumeStats()
    B.check(B.load_library().amemPauseResumeStatsGet(None, ctypes.byref(s)), "amemPauseResumeStatsGet")
    return B.struct_to_dict(s)


def inject(what: str, nth: int = 1, param: int = 0) -> None:
    B.check(B.load_library().amemInject(what.encode(), nth, param), "amemInject")


def group_start() -> None:
    B.check(B.load_library().ncclGroupStart(), "ncclGroupStart")


def group_end() -> None:
    B.check(B.load_library().ncclGroupEnd(), "ncclGroupEnd")


def mem_alloc(nbytes: int) -> int:
    p = ctypes.c_void_p()
    B.check(B.load_library().ncclMemAlloc(ctypes.byref(p), nbytes), "ncclMemAlloc")
    return p.value


def mem_free(ptr: int) -> None:
    B.check(B.load_library().ncclMemFree(ctypes.c_void_p(ptr)), "ncclMemFree")


class _RawBuffer:
    """Lets torch view device memory that the library allocated (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class Window:
    """Memory from ``ncclMemAlloc`` registered with a communicator (``ncclCommWindowRegister``):
    every rank maps it, all-reduces whose buffers lie inside run in place, and it is saved,
    released and restored with the communicator on pause / resume.

    Reference parity: the allocations the reference tracks for NCCL's symmetric windows and
    registered user buffers (nccl_patch/nccl_2.27.5-1.diff:56-58, 630-632)."""

    def __init__(self, comm: "Communicator", ptr: int, nbytes: int, handle: int, owns: bool):
        self.comm, self.ptr, self.nbytes, self._h, self._owns = comm, ptr, nbytes, handle, owns

    def tensor(self, dtype=None, numel: Optional[int] = None, offset_bytes: int = 0):
        """A torch view of (part of) this rank's window memory (CUDA backend) or a numpy view
        (mock backend)."""
        if self.comm.lib.amemBackendIsDevice():
            torch = _torch()
            t = torch.as_tensor(_RawBuffer(self.ptr + offset_bytes, self.nbytes - offset_bytes), device="cuda")
            if dtype is not None:
                t = t.view(dtype)
            return t if numel is None else t[:numel]
        import numpy as np
        buf = (ctypes.c_ubyte * (self.nbytes - offset_bytes)).from_address(self.ptr + offset_bytes)
        arr = np.frombuffer(buf, dtype=np.uint8)
        if dtype is not None:
            arr = arr.view(dtype)
        return arr if numel is None else arr[:numel]

    def free(self) -> None:
        """Collective: deregisters the window and, if it was made by ``window_alloc``, frees it."""
        if self._h:
            B.check(self.comm.lib.ncclCommWindowDeregister(self.comm._h, ctypes.c_void_p(self._h)), "ncclCommWindowDeregister")
            self._h = 0
            if self._owns:
                mem_free(self.ptr)


class Communicator:
    """A rank's handle on a communicator (``ncclComm_t``)."""

    def __init__(self, nranks: int, rank: int, unique_id: bytes, _handle: Optional[int] = None):
        self.lib = B.load_library()
        self.nranks, self.rank = nranks, rank
        if _handle is not None:
            self._h = ctypes.c_void_p(_handle)
            return
        uid = B.UniqueId.from_buffer_copy(unique_id)
        h = ctypes.c_void_p()
        B.check(self.lib.ncclCommInitRank(ctypes.byref(h), nranks, uid, rank), "ncclCommInitRank")
        self._h = h

    # -- construction helpers -----------------------------------------------------------
    @classmethod
    def from_torch_distributed(cls, group=None) -> "Communicator":
        """Bootstraps through an initialised torch.distributed group (any backend): rank 0
        creates the unique id and the group broadcasts it."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [get_unique_id() if rank == 0 else None]
        src = dist.get_global_rank(group, 0) if group is not None else 0
        dist.broadcast_object_list(box, src=src, group=group)
        return cls(world, rank, box[0])

    def split(self, color: int, key: int = 0) -> Optional["Communicator"]:
        h = ctypes.c_void_p()
        B.check(self.lib.ncclCommSplit(self._h, color, key, ctypes.byref(h), None), "ncclCommSplit")
        if not h.value:
            return None
        n, r = ctypes.c_int(), ctypes.c_int()
        self.lib.ncclCommCount(h, ctypes.byref(n))
        self.lib.ncclCommUserRank(h, ctypes.byref(r))
        return Communicator(n.value, r.value, b"", _handle=h.value)

    def shrink(self, exclude) -> "Communicator":
        """A new communicator over the ranks of this one that are not in ``exclude``
        (ncclCommShrink).  Only the surviving ranks call it; the excluded ones may be gone."""
        ex = (ctypes.c_int * max(1, len(exclude)))(*exclude)
        h = ctypes.c_void_p()
        B.check(self.lib.ncclCommShrink(self._h, ex, len(exclude), ctypes.byref(h), None, 0), "ncclCommShrink")
        n, r = ctypes.c_int(), ctypes.c_int()
        self.lib.ncclCommCount(h, ctypes.byref(n))
        self.lib.ncclCommUserRank(h, ctypes.byref(r))
        return Communicator(n.value, r.value, b"", _handle=h.value)

    @property
    def handle(self) -> int:
        return self._h.value

    def window_register(self, ptr: int, nbytes: int, _owns: bool = False) -> Window:
        """Collective: registers memory from :func:`mem_alloc` as a window of this communicator."""
        w = ctypes.c_void_p()
        B.check(self.lib.ncclCommWindowRegister(self._h, ctypes.c_void_p(ptr), ctypes.c_size_t(nbytes), ctypes.byref(w), 0), "ncclCommWindowRegister")
        return Window(self, ptr, nbytes, w.value, _owns)

    def window_alloc(self, nbytes: int) -> Window:
        """Collective: ``ncclMemAlloc`` + ``ncclCommWindowRegister``; same size on every rank."""
        return self.window_register(mem_alloc(nbytes), nbytes, _owns=True)

    def info(self) -> dict:
        emu, nvls, stage = ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()
        B.check(self.lib.amemCommInfo(self._h, ctypes.byref(emu), ctypes.byref(nvls), ctypes.byref(stage)), "amemCommInfo")
        return {"emulated": bool(emu.value), "nvls": bool(nvls.value), "stage_bytes": stage.value}

    def check_canary(self) -> None:
        """Raises if a kernel wrote past the staging layout (guard enabled with AMEM_CANARY=1)."""
        B.check(self.lib.amemCheckCanary(self._h), "amemCheckCanary")

    def destroy(self) -> None:
        if self._h is not None and self._h.value:
            B.check(self.lib.ncclCommDestroy(self._h), "ncclCommDestroy")
            self._h = None

    def abort(self) -> None:
        if self._h is not None and self._h.value:
            self.lib.ncclCommAbort(self._h)
            self._h = None

    def async_error(self) -> int:
        e = ctypes.c_int()
        B.check(self.lib.ncclCommGetAsyncError(self._h, ctypes.byref(e)), "ncclCommGetAsyncError")
        return e.value

    # -- collectives --------------------------------------------------------------------
    def all_reduce(self, send, recv=None, op: str = "sum", stream=None, algo: str = "auto"):
        recv = send if recv is None else recv
        st = _stream_handle(stream, send)
        if algo == "auto":
            rc = self.lib.ncclAllReduce(_ptr(send), _ptr(recv), _numel(send), _dtype_code(send), B.OPS[op], self._h, st)
        else:
            rc = self.lib.amemAllReduceAlgo(_ptr(send), _ptr(recv), _numel(send), _dtype_code(send), B.OPS[op], B.ALGOS[algo], self._h, st)
        B.check(rc, "ncclAllReduce")
        return recv

    def reduce(self, send, recv=None, root: int = 0, op: str = "sum", stream=None):
        recv = send if recv is None else recv
        B.check(self.lib.ncclReduce(_ptr(send), _ptr(recv), _numel(send), _dtype_code(send), B.OPS[op], root, self._h,
                                    _stream_handle(stream, send)), "ncclReduce")
        return recv

    def broadcast(self, send, recv=None, root: int = 0, stream=None):
        recv = send if recv is None else recv
        B.check(self.lib.ncclBroadcast(_ptr(send), _ptr(recv), _numel(send), _dtype_code(send), root, self._h,
                                       _stream_handle(stream, send)), "ncclBroadcast")
        return recv

    def all_gather(self, send, recv, stream=None):
        assert _numel(recv) == _numel(send) * self.nranks
        B.check(self.lib.ncclAllGather(_ptr(send), _ptr(recv), _numel(send), _dtype_code(send), self._h,
                                       _stream_handle(stream, send)), "ncclAllGather")
        return recv

    def reduce_scatter(self, send, recv, op: str = "sum", stream=None, scale: Optional[float] = None):
        """recv = reduce over ranks of send's rank-th slice.  With ``scale`` or when the dtypes
        differ the fused scale+cast kernel is used (sum only)."""
        assert _numel(send) == _numel(recv) * self.nranks
        st = _stream_handle(stream, send)
        if scale is None and _dtype_code(send) == _dtype_code(recv):
            rc = self.lib.ncclReduceScatter(_ptr(send), _ptr(recv), _numel(recv), _dtype_code(send), B.OPS[op], self._h, st)
        else:
            if op not in ("sum",):
                raise ValueError("fused scale/cast reduce-scatter supports op='sum' only")
            rc = self.lib.amemReduceScatterScaleCast(_ptr(send), _ptr(recv), _numel(recv), _dtype_code(send), _dtype_code(recv),
                                                     1.0 if scale is None else float(scale), self._h, st)
        B.check(rc, "ncclReduceScatter")
        return recv

    def all_to_all(self, send, recv, stream=None):
        assert _numel(send) == _numel(recv) and _numel(send) % self.nranks == 0
        B.check(self.lib.ncclAlltoAll(_ptr(send), _ptr(recv), _numel(send) // self.nranks, _dtype_code(send), self._h,
                                      _stream_handle(stream, send)), "ncclAlltoAll")
        return recv

    def all_to_all_v(self, send, recv, send_counts, recv_counts, send_displs=None, recv_displs=None, stream=None):
        """Variable-size all-to-all (element counts / displacements per peer, MPI_Alltoallv
        style): one grouped launch of sends and receives -- the form in which NCCL applications
        write it (ncclGroupStart + ncclSend/ncclRecv per peer + ncclGroupEnd); this rank's own
        block is a local copy.  Counts must match pairwise: send_counts[j] here equals
        recv_counts[me] on rank j."""
        n, me = self.nranks, self.rank
        assert len(send_counts) == n and len(recv_counts) == n and send.dtype == recv.dtype
        def displs(counts, given):
            if given is not None:
                return list(given)
            out, acc = [], 0
            for c in counts:
                out.append(acc)
                acc += int(c)
            return out
        sd, rd = displs(send_counts, send_displs), displs(recv_counts, recv_displs)
        if int(send_counts[me]) != int(recv_counts[me]):
            raise ValueError("all_to_all_v: this rank's own send and receive counts differ")
        arr = lambda v: (ctypes.c_size_t * n)(*[int(x) for x in v])  # noqa: E731
        B.check(self.lib.amemAlltoAllv(_ptr(send), arr(send_counts), arr(sd), _ptr(recv), arr(recv_counts), arr(rd),
                                       _dtype_code(send), self._h, _stream_handle(stream, send)), "amemAlltoAllv")
        return recv

    def send(self, tensor, peer: int, stream=None):
        B.check(self.lib.ncclSend(_ptr(tensor), _numel(tensor), _dtype_code(tensor), peer, self._h, _stream_handle(stream, tensor)), "ncclSend")

    def recv(self, tensor, peer: int, stream=None):
        B.check(self.lib.ncclRecv(_ptr(tensor), _numel(tensor), _dtype_code(tensor), peer, self._h, _stream_handle(stream, tensor)), "ncclRecv")

    # -- pause / resume -----------------------------------------------------------------
    def pause(self) -> None:
        h = ctypes.c_void_p(self._h.value)
        B.check(self.lib.ncclPause(ctypes.byref(h)), "ncclPause")

    def resume(self) -> None:
        h = ctypes.c_void_p(self._h.value)
        B.check(self.lib.ncclResume(ctypes.byref(h)), "ncclResume")

    def pause_resume_stats(self) -> dict:
        s = B.PauseResumeStats()
        B.check(self.lib.amemPauseResumeStatsGet(self._h, ctypes.byref(s)), "amemPauseResumeStatsGet")
        return B.struct_to_dict(s)
