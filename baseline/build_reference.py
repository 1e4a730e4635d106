"""Builds the reference arm: the reference's plugin, unchanged, plus the harness that drives it.

The reference is a C++ plugin (``amem_nccl_plugin/``) plus a patch for NCCL 2.27.5.  The patched
NCCL cannot be built offline (its NCCL and nccl-tests submodules are empty), but the plugin — the
part that tracks allocations and implements pause / resume — needs only ``cuda.h``,
``cuda_runtime.h`` and ``nccl.h`` (for a few typedefs).  This script follows the reference's own
recipe (amem_nccl_plugin/Makefile:27-34: eight ``g++ -c`` objects, one ``nvcc -shared`` link with
``-soname libamem_nccl.so.1``) on a scratch copy of the sources, since the source tree itself may
be read-only, and writes

    baseline/_ref/lib/libamem_nccl.so.1     the reference plugin
    baseline/_ref/lib/libref_harness.so     baseline/ref_harness.cc, linked against it
    baseline/_ref/BUILD_INFO.json           what was built from where

``baseline/_ref`` is not tracked.  The reference sources are looked for in ``$AMEM_REFERENCE_SRC``
and then in ``reference/`` beside the repository.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
LIB_DIR = REF_OUT / "lib"
PLUGIN_SO = LIB_DIR / "libamem_nccl.so.1"
HARNESS_SO = LIB_DIR / "libref_harness.so"
INFO = REF_OUT / "BUILD_INFO.json"

# object list of the reference's Makefile (amem_nccl_plugin/Makefile:28)
OBJECTS = ["amem_nccl", "gmm_common_impl", "gmm_client_cfg", "gmm_client_impl", "gmm_server_impl", "gmm_worker_impl",
           "gmm_host_shm_impl", "gmm_api_stats"]


def reference_source() -> Path | None:
    cands = []
    if os.environ.get("AMEM_REFERENCE_SRC"):
        cands.append(Path(os.environ["AMEM_REFERENCE_SRC"]))
    cands.append(HERE.parent.parent / "reference")
    for c in cands:
        if (c / "amem_nccl_plugin" / "amem_nccl.cpp").exists():
            return c
    return None


def _run(cmd: list[str], cwd: Path) -> None:
    res = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)} failed:\n{res.stdout}\n{res.stderr}")


def _tree_digest(d: Path) -> str:
    h = hashlib.sha256()
    for p in sorted(d.iterdir()):
        if p.suffix in (".cpp", ".h") or p.name == "Makefile":
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()[:16]


def build(force: bool = False) -> dict:
    """Returns the build record; ``{"available": False, "why": ...}`` when nothing can be built."""
    src = reference_source()
    if src is None:
        if PLUGIN_SO.exists() and HARNESS_SO.exists() and INFO.exists():
            return json.loads(INFO.read_text())   # built earlier, sources not on this machine
        return {"available": False, "why": "reference sources not found and no earlier build under baseline/_ref"}
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    nvcc = shutil.which("nvcc") or str(cuda / "bin" / "nvcc")
    digest = _tree_digest(src / "amem_nccl_plugin")
    harness_src = HERE / "ref_harness.cc"
    if not force and PLUGIN_SO.exists() and HARNESS_SO.exists() and INFO.exists():
        info = json.loads(INFO.read_text())
        if info.get("plugin_sources_sha") == digest and HARNESS_SO.stat().st_mtime >= harness_src.stat().st_mtime:
            return info
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    nccl_inc = "/usr/include" if Path("/usr/include/nccl.h").exists() else str(HERE.parent / "csrc" / "include")
    with tempfile.TemporaryDirectory(prefix="amem_ref_build_") as tmp:
        work = Path(tmp) / "amem_nccl_plugin"
        shutil.copytree(src / "amem_nccl_plugin", work)
        flags = [f"-I{nccl_inc}", f"-I{cuda}/include", "-D_GNU_SOURCE", "-g", "-O2", "-DNDEBUG", "-std=c++17"]
        for o in OBJECTS:
            _run(["g++", "-c", "-g", "-o", f"{o}.o", f"{o}.cpp", "-fPIC", *flags], work)
        _run([nvcc, "-o", str(PLUGIN_SO), *[f"{o}.o" for o in OBJECTS], f"-L{cuda}/lib64", "-shared", "-lrt", "-ldl", "-lpthread",
              "-Xcompiler", "-fPIC", "-Xlinker", "-soname,libamem_nccl.so.1", "-lcuda", "-lcudart",
              "-gencode", "arch=compute_100a,code=sm_100a"], work)
        _run(["g++", "-shared", "-fPIC", "-O2", "-std=c++17", "-o", str(HARNESS_SO), str(harness_src), f"-I{work}", f"-I{nccl_inc}",
              f"-I{cuda}/include", f"-L{LIB_DIR}", "-l:libamem_nccl.so.1", f"-L{cuda}/lib64", f"-L{cuda}/lib64/stubs", "-lcuda", "-lcudart",
              "-Wl,-rpath,$ORIGIN"], work)
    info = {"available": True, "plugin": str(PLUGIN_SO.relative_to(HERE.parent)), "harness": str(HARNESS_SO.relative_to(HERE.parent)),
            "plugin_sources_sha": digest, "objects": OBJECTS,
            "recipe": "amem_nccl_plugin/Makefile:27-34 (g++ -c per object, nvcc -shared, sm_100a only), sources unchanged"}
    INFO.write_text(json.dumps(info, indent=1))
    return info


if __name__ == "__main__":
    print(json.dumps(build(force=True), indent=1))
