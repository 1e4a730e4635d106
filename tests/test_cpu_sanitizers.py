"""Host runtime under ThreadSanitizer and AddressSanitizer + UBSan.

The registry, the mock VMM backend, the Unix-socket mesh and the pause / resume engine are
compiled (g++, no CUDA) together with tests/native/engine_stress.cc, which runs several ranks as
threads through pause / resume cycles with real descriptor passing and shared pages.  Any report
of the sanitizers fails the test (halt_on_error / exitcode); device code cannot be covered this
way, its bounded waits and index checks are covered by the GPU suite instead."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCES = ["tests/native/engine_stress.cc", "csrc/vmm/registry.cc", "csrc/vmm/mock_backend.cc", "csrc/vmm/pause_resume.cc",
           "csrc/ipc/uds.cc", "csrc/ipc/rendezvous.cc"]


def _build(tmp_path, name, flags):
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("g++ not available")
    exe = tmp_path / name
    cmd = [gxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, *[os.path.join(ROOT, s) for s in SOURCES],
           "-o", str(exe), "-lpthread", "-lrt"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if res.returncode != 0 and ("cannot find -l" in res.stderr or "unrecognized" in res.stderr):
        pytest.skip("this toolchain has no runtime for " + " ".join(flags))
    assert res.returncode == 0, res.stderr[-4000:]
    return exe


@pytest.mark.parametrize("name,flags,env", [
    ("stress_tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1 exitcode=66"}),
    ("stress_asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"],
     {"ASAN_OPTIONS": "detect_leaks=1:halt_on_error=1", "UBSAN_OPTIONS": "print_stacktrace=1"}),
])
def test_engine_stress_is_clean_under_sanitizers(tmp_path, name, flags, env):
    exe = _build(tmp_path, name, flags)
    run_env = dict(os.environ, GMM_IPC_DIR=str(tmp_path), GMM_LOG="2", **env)
    res = subprocess.run([str(exe), "4", "8"], capture_output=True, text=True, timeout=600, env=run_env)
    assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-6000:])
    assert "engine stress ok" in res.stdout
    assert "WARNING: ThreadSanitizer" not in res.stderr and "ERROR: AddressSanitizer" not in res.stderr and "runtime error" not in res.stderr
