"""Reference arm of the headline benchmark: the unmodified reference plugin, one process per GPU.

What the reference's patched NCCL would do at communicator set-up is replayed through
``libref_harness.so`` (baseline/ref_harness.cc): every rank creates its allocations with the CUDA
virtual-memory calls and reports them with ``amem_addAllocInfo``; every peer imports the shared
ones and reports the import with the exporter's handle value, which is what lets the reference's
worker thread on the exporter record who mapped what (amem_nccl_plugin/amem_nccl.cpp:102-269,
297-329).  ``pause()`` / ``resume()`` are ``amem_memPause`` / ``amem_memResume``
(amem_nccl_plugin/amem_nccl.cpp:467-677), the bodies of the reference's ncclPause / ncclResume.

The layout mirrors this library's at the same footprint: ``records`` shared allocations of
``shared_bytes`` in total, each imported by every other rank (what this library's staging segment
is, and what NCCL's p2p buffers are in the reference: caller tag 1), plus one private allocation of
``stateful_bytes`` (an ncclMemAlloc buffer, caller tag 3).  The reference saves and restores all
of it; that is its stock behaviour.

File descriptors cross the process boundary here, on datagram Unix sockets (the reference gets
them from NCCL's bootstrap, which is not part of the plugin).
"""
from __future__ import annotations

import array
import ctypes
import os
import socket
import struct
import tempfile
import threading
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_DIR = HERE / "_ref" / "lib"
_MSG = struct.Struct("<iiQQ")   # source rank, record index, size, exporter handle value


def available() -> tuple[bool, str]:
    for name in ("libamem_nccl.so.1", "libref_harness.so"):
        if not (LIB_DIR / name).exists():
            return False, f"baseline/_ref/lib/{name} is missing (python baseline/build_reference.py builds it where the reference sources are)"
    return True, ""


def restrict_visible_devices(world: int) -> None:
    """The reference waits until every VISIBLE GPU has a participating process
    (amem_nccl_plugin/gmm_client_impl.cpp:182-187), so each rank must see exactly the job's GPUs.
    Must run before CUDA is initialised in this process."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    devs = [d for d in vis.split(",") if d.strip()] if vis else [str(i) for i in range(world)]
    os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(devs[:world])


def point_reference_at_libcuda() -> None:
    """The plugin dlopen()s libcuda.so.1 from two fixed directories unless CUDA_LIB_PATH names the
    file (amem_nccl_plugin/gmm_client_cfg.cpp:33-37) and aborts when it finds none; container images
    keep the driver library elsewhere.  The path the dynamic loader actually resolves is taken from
    this process's own mappings."""
    if os.environ.get("CUDA_LIB_PATH"):
        return
    try:
        ctypes.CDLL("libcuda.so.1")
        with open("/proc/self/maps") as f:
            for line in f:
                path = line.split()[-1]
                if "libcuda.so" in path and os.path.exists(path):
                    os.environ["CUDA_LIB_PATH"] = path
                    return
    except OSError:
        pass


class ReferenceArm:
    def __init__(self, rank: int, world: int, local: int, shared_bytes: int, records: int, stateful_bytes: int, barrier):
        self.rank, self.world, self.local = rank, world, local
        self.barrier = barrier
        os.environ["AMEM_ENABLE"] = "1"            # the plugin is off unless asked (amem_nccl.cpp:711)
        os.environ.setdefault("GMM_LOG", "3")
        point_reference_at_libcuda()
        # the plugin first, so that the harness resolves against this exact file
        self.plugin = ctypes.CDLL(str(LIB_DIR / "libamem_nccl.so.1"), mode=ctypes.RTLD_GLOBAL)
        self.h = ctypes.CDLL(str(LIB_DIR / "libref_harness.so"))
        self.h.rh_last_error.restype = ctypes.c_char_p
        self.h.rh_granularity.restype = ctypes.c_uint64
        self.h.rh_alloc_local.argtypes = [ctypes.c_uint64, ctypes.c_int, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        self.h.rh_export.argtypes = [ctypes.c_uint64, ctypes.POINTER(ctypes.c_int)]
        self.h.rh_import.argtypes = [ctypes.c_int, ctypes.c_uint64, ctypes.c_int, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64)]
        self.h.rh_fill.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32]
        self.h.rh_check.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32]
        self.h.rh_mem_info.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        # every rank has loaded the plugin (its constructor deletes other processes' socket files,
        # amem_nccl.cpp:708) before anybody creates one
        barrier()
        self._ck(self.h.rh_init(local), "rh_init")
        gran = int(self.h.rh_granularity())
        rnd = lambda b: max(gran, (int(b) + gran - 1) // gran * gran)  # noqa: E731
        self.shared = []      # (ptr, size, handle)
        self.private = []     # (ptr, size)
        self.imported = []    # (ptr, size, source rank, record index)
        each = rnd(shared_bytes // max(1, records)) if shared_bytes else 0
        for _ in range(records if each else 0):
            p, hd = ctypes.c_uint64(), ctypes.c_uint64()
            self._ck(self.h.rh_alloc_local(each, 1, ctypes.byref(p), ctypes.byref(hd)), "rh_alloc_local")   # the first call boots the control plane
            self.shared.append((p.value, each, hd.value))
        if stateful_bytes:
            p, hd = ctypes.c_uint64(), ctypes.c_uint64()
            sz = rnd(stateful_bytes)
            self._ck(self.h.rh_alloc_local(sz, 3, ctypes.byref(p), ctypes.byref(hd)), "rh_alloc_local")
            self.private.append((p.value, sz))
        if world > 1 and self.shared:
            self._exchange()
        barrier()

    def _ck(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what}: {self.h.rh_last_error().decode()}")

    def _exchange(self) -> None:
        ipc = os.path.join(tempfile.gettempdir(), f"amemref_{os.environ.get('MASTER_PORT', '0')}")
        os.makedirs(ipc, exist_ok=True)
        path = lambda r: os.path.join(ipc, f"r{r}.sock")  # noqa: E731
        sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
        if os.path.exists(path(self.rank)):
            os.unlink(path(self.rank))
        sock.bind(path(self.rank))
        sock.settimeout(120)
        self.barrier()
        expect = len(self.shared) * (self.world - 1)
        got = []

        def receiver():
            for _ in range(expect):
                data, fds, _f, _a = socket.recv_fds(sock, _MSG.size, 1)
                got.append((_MSG.unpack(data), fds[0]))

        th = threading.Thread(target=receiver)
        th.start()
        out = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
        for idx, (_p, size, handle) in enumerate(self.shared):
            fd = ctypes.c_int(-1)
            self._ck(self.h.rh_export(handle, ctypes.byref(fd)), "rh_export")
            for r in range(self.world):
                if r != self.rank:
                    # (socket.send_fds drops its address argument: sendmsg directly)
                    out.sendmsg([_MSG.pack(self.rank, idx, size, handle)], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd.value]))], 0, path(r))
            os.close(fd.value)
        th.join()
        out.close()
        sock.close()
        for (src, idx, size, handle), fd in sorted(got, key=lambda g: g[0][:2]):
            p = ctypes.c_uint64()
            # device index of the exporter among the visible devices == its local rank
            self._ck(self.h.rh_import(fd, size, src, handle, ctypes.byref(p)), "rh_import")
            self.imported.append((p.value, size, src, idx))

    @staticmethod
    def pattern(rank: int, idx: int, step: int) -> int:
        return (0x5A000000 | ((rank & 0xF) << 20) | ((idx & 0x3FF) << 8) | (step & 0xFF)) & 0xFFFFFFFF

    def touch(self, step: int) -> None:
        """Every tracked local allocation gets this step's pattern."""
        for idx, (p, size, _h) in enumerate(self.shared):
            self._ck(self.h.rh_fill(p, size, self.pattern(self.rank, idx, step)), "rh_fill")
        for p, size in self.private:
            self._ck(self.h.rh_fill(p, size, self.pattern(self.rank, 1023, step)), "rh_fill")

    def verify(self, step: int) -> int:
        """Words that differ from the pattern after resume: own allocations and, through the
        re-imported mappings, the peers'."""
        bad = 0
        for idx, (p, size, _h) in enumerate(self.shared):
            bad += max(0, self.h.rh_check(p, size, self.pattern(self.rank, idx, step)))
        for p, size in self.private:
            bad += max(0, self.h.rh_check(p, size, self.pattern(self.rank, 1023, step)))
        for p, size, src, idx in self.imported:
            bad += max(0, self.h.rh_check(p, size, self.pattern(src, idx, step)))
        return bad

    def mem_free(self) -> int:
        f, t = ctypes.c_uint64(), ctypes.c_uint64()
        self._ck(self.h.rh_mem_info(ctypes.byref(f), ctypes.byref(t)), "rh_mem_info")
        return f.value

    def pause(self) -> None:
        rc = self.h.rh_pause()
        if rc != 0:
            raise RuntimeError(f"amem_memPause returned {rc}")

    def resume(self) -> None:
        rc = self.h.rh_resume()
        if rc != 0:
            raise RuntimeError(f"amem_memResume returned {rc}")

    def tracked_bytes(self) -> dict:
        return {"local_records": len(self.shared) + len(self.private), "imported_records": len(self.imported),
                "local_bytes": sum(s for _p, s, _h in self.shared) + sum(s for _p, s in self.private),
                "imported_bytes": sum(s for _p, s, _r, _i in self.imported)}
