"""Multi-process, multi-GPU correctness: one rank per GPU under torch.distributed.run, on real peer
mappings, the NVLink multicast paths included (tests/multigpu_check.py does the checking).  Runs
when the machine shows at least two GPUs; skipped on a single-GPU machine, where the emulated-rank
tests cover the protocols."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_all_checks_one_rank_per_gpu():
    n = min(8, torch.cuda.device_count())
    n = 8 if n == 8 else 4 if n >= 4 else 2
    env = dict(os.environ)
    env.pop("AMEM_CANARY", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "multigpu_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    tail = "\n".join(res.stdout.splitlines()[-40:]) + "\n" + "\n".join(res.stderr.splitlines()[-20:])
    assert res.returncode == 0 and "ALL OK" in res.stdout, tail
