"""ctypes bindings of ``libamem_b200.so`` (pynccl-style).

The reference documents exactly this integration style for SGLang's ``pynccl`` wrapper: load
the library, look ``ncclPause`` / ``ncclResume`` / ``ncclSetGroupID`` up by name and call them
with a communicator handle (README.md:262-294 of the reference).  The same names are exported
here, next to the usual NCCL entry points, so such a wrapper can point at this library.

Buffers are passed as raw addresses: CUDA tensors with the CUDA backend, CPU tensors or numpy
arrays with the mock backend (``AMEM_BACKEND=mock``) whose "device memory" is host memory.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libamem_b200.so"

ncclSuccess = 0
RESULT_NAMES = {
    0: "ncclSuccess", 1: "ncclUnhandledCudaError", 2: "ncclSystemError", 3: "ncclInternalError",
    4: "ncclInvalidArgument", 5: "ncclInvalidUsage", 6: "ncclRemoteError", 7: "ncclInProgress",
}
# ncclDataType_t / ncclRedOp_t
DTYPES = {"int8": 0, "uint8": 1, "int32": 2, "uint32": 3, "int64": 4, "uint64": 5,
          "float16": 6, "float32": 7, "float64": 8, "bfloat16": 9,
          "float8_e4m3fn": 10, "float8_e5m2": 11}   # 8-bit floats: copy collectives only
OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}
ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3, "window": 4}


class NcclError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str):
        self.code = code
        super().__init__(f"{where}: {RESULT_NAMES.get(code, code)}: {detail}")


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


class MemStats(ctypes.Structure):
    _fields_ = [("bytes_by_tag", ctypes.c_uint64 * 16),
                ("stateful_bytes", ctypes.c_uint64), ("scratch_bytes", ctypes.c_uint64),
                ("imported_bytes", ctypes.c_uint64), ("multicast_bytes", ctypes.c_uint64),
                ("live_bytes", ctypes.c_uint64), ("paused_bytes", ctypes.c_uint64), ("shadow_bytes", ctypes.c_uint64),
                ("n_local", ctypes.c_uint64), ("n_imported", ctypes.c_uint64),
                ("pause_count", ctypes.c_uint64), ("resume_count", ctypes.c_uint64),
                ("group_id", ctypes.c_int), ("paused", ctypes.c_int)]


class PauseResumeStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_double) for n in (
        "quiesce_us", "offload_us", "release_import_us", "release_local_us", "pause_barrier_us", "pause_total_us",
        "create_map_us", "agree_us", "exchange_us", "import_us", "preload_us", "resume_barrier_us", "resume_total_us")] + \
        [(n, ctypes.c_uint64) for n in (
            "bytes_offloaded", "bytes_preloaded", "bytes_released_local", "bytes_released_peer",
            "n_offload", "n_release_local", "n_release_peer",
            "free_before_pause", "free_after_pause", "free_after_resume")]


def struct_to_dict(s: ctypes.Structure) -> dict:
    out = {}
    for name, _ in s._fields_:
        v = getattr(s, name)
        out[name] = list(v) if hasattr(v, "__len__") else v
    return out


def library_path() -> Path:
    return Path(os.environ.get("AMEM_LIBRARY", str(_LIB_PATH)))


def load_library(build_if_missing: bool = True) -> ctypes.CDLL:
    """Loads (building first if the shared object is missing) and annotates the library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        if not build_if_missing:
            raise FileNotFoundError(f"{path} is missing; run python -m asystem_amem_b200._build")
        from . import _build
        _build.build()
    # RTLD_LOCAL: the nccl* names must not shadow (or be shadowed by) the NCCL inside torch.
    lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)
    c_void_p, c_size_t, c_int = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    P = ctypes.POINTER
    sig = {
        "ncclGetVersion": [P(c_int)],
        "ncclGetUniqueId": [P(UniqueId)],
        "ncclCommInitRank": [P(c_void_p), c_int, UniqueId, c_int],
        "ncclCommDestroy": [c_void_p],
        "ncclCommAbort": [c_void_p],
        "ncclCommFinalize": [c_void_p],
        "ncclCommSplit": [c_void_p, c_int, c_int, P(c_void_p), c_void_p],
        "ncclCommShrink": [c_void_p, P(c_int), c_int, P(c_void_p), c_void_p, c_int],
        "ncclCommGetAsyncError": [c_void_p, P(c_int)],
        "ncclCommCount": [c_void_p, P(c_int)],
        "ncclCommCuDevice": [c_void_p, P(c_int)],
        "ncclCommUserRank": [c_void_p, P(c_int)],
        "ncclMemAlloc": [P(c_void_p), c_size_t],
        "ncclMemFree": [c_void_p],
        "ncclAllReduce": [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p],
        "amemAllReduceAlgo": [c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p],
        "ncclReduce": [c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p],
        "ncclBroadcast": [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p],
        "ncclReduceScatter": [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p],
        "amemReduceScatterScaleCast": [c_void_p, c_void_p, c_size_t, c_int, c_int, ctypes.c_float, c_void_p, c_void_p],
        "ncclAllGather": [c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p],
        "ncclAlltoAll": [c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p],
        "ncclSend": [c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p],
        "ncclRecv": [c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p],
        "ncclGroupStart": [],
        "ncclGroupEnd": [],
        "ncclPause": [P(c_void_p)],
        "ncclResume": [P(c_void_p)],
        "ncclMemStats": [],
        "ncclSetGroupID": [c_int],
        "ncclGetGroupID": [P(c_int)],
        "amemMemStatsGet": [P(MemStats)],
        "amemPauseResumeStatsGet": [c_void_p, P(PauseResumeStats)],
        "amemCommInfo": [c_void_p, P(c_int), P(c_int), P(c_size_t)],
        "amemInject": [ctypes.c_char_p, c_int, c_int],
        "amemAlltoAllv": [c_void_p, P(c_size_t), P(c_size_t), c_void_p, P(c_size_t), P(c_size_t), c_int, c_void_p, c_void_p],
        "amemCheckCanary": [c_void_p],
        "amemDebugDirtyCanary": [c_void_p],
        "amemBackendUsage": [P(c_size_t), P(c_size_t), P(ctypes.c_char_p)],
        "amemBackendIsDevice": [],
        "ncclCommWindowRegister": [c_void_p, c_void_p, c_size_t, P(c_void_p), c_int],
        "ncclCommWindowDeregister": [c_void_p, c_void_p],
        "amemMoeBuffers": [c_void_p, c_int, c_int, P(c_void_p), P(c_void_p)],
        "amemMoeDispatch": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "amemMoeDispatchCounted": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "amemMoeCombine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "amemGemmBf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "amemGemmPlan": [c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)],
        "amemAllGatherGemmPlan": [c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)],
        "amemDeviceWaitProbe": [c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(ctypes.c_float)],
        "amemGroupedGemmBf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "amemAllGatherGemm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
        "amemGemmReduceScatter": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.amemLastError.restype = ctypes.c_char_p
    lib.amemLastError.argtypes = []
    lib.ncclGetErrorString.restype = ctypes.c_char_p
    lib.ncclGetErrorString.argtypes = [c_int]
    _LIB = lib
    return lib


def check(code: int, where: str) -> None:
    if code != ncclSuccess:
        detail = load_library().amemLastError()
        raise NcclError(code, where, detail.decode(errors="replace") if detail else "")
