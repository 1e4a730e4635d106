"""In-tree build of the native library (``lib/libamem_b200.so``).

Every source under ``csrc/`` is compiled by nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``) and linked with the static CUDA
runtime into one shared object that sits inside the Python package, so a source checkout
that was built once can be shipped to a GPU machine as is.  The build is incremental
(object files under ``build/`` are reused while they are newer than every source and header).

Run ``python -m asystem_amem_b200._build`` or call :func:`build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ_DIR = ROOT / "build" / "obj"
LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB_PATH = LIB_DIR / "libamem_b200.so"

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-DAMEM_WITH_NVTX", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function,-fvisibility=default"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources() -> list[Path]:
    out = []
    for pat in ("*.cc", "*.cu"):
        out += sorted(CSRC.rglob(pat))
    return out


def _headers_mtime() -> float:
    newest = 0.0
    for pat in ("*.h", "*.cuh", "*.inl"):
        for p in CSRC.rglob(pat):
            newest = max(newest, p.stat().st_mtime)
    return newest


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> None:
    cmd = [nvcc, *GENCODE, *COMMON, "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cu" and os.environ.get("AMEM_PTXAS_V"):
        cmd += ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if os.environ.get("AMEM_PTXAS_V") and res.stderr:
        print(res.stderr, file=sys.stderr)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what is stale and link the shared library.  Returns its path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    hdr_time = _headers_mtime()
    jobs = []
    objs = []
    for src in sources():
        rel = src.relative_to(CSRC)
        obj = OBJ_DIR / ("_".join(rel.with_suffix("").parts) + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        workers = min(len(jobs), os.cpu_count() or 4)
        with ThreadPoolExecutor(max_workers=workers) as pool:
            list(pool.map(lambda j: _compile_one(nvcc, j[0], j[1], verbose), jobs))
    need_link = force or bool(jobs) or not LIB_PATH.exists() or any(o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs)
    if need_link:
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, *GENCODE, "-shared", "-cudart", "static", "-o", str(tmp), *map(str, objs),
               "-Xlinker", "-Bsymbolic", "-lpthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
