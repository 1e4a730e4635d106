"""A device-side wait that runs out: the kernel records an error in host-visible status words and
returns, the CUDA context stays usable.  The wait is made to run out on purpose the harmless way:
a flag that nothing sets and a limit of a fraction of a second (no trap, no bad address, no
endless loop)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_reports_a_status_and_leaves_the_context_usable():
    from asystem_amem_b200.bindings import load_library
    lib = load_library()
    code, ms = ctypes.c_int(-1), ctypes.c_float(0.0)
    # the flag is there: no error, no waiting (the first call also loads the kernel: not timed)
    assert lib.amemDeviceWaitProbe(300, 1, ctypes.byref(code), ctypes.byref(ms)) == 0 and code.value == 0
    assert lib.amemDeviceWaitProbe(300, 1, ctypes.byref(code), ctypes.byref(ms)) == 0
    assert code.value == 0 and ms.value < 200.0, (code.value, ms.value)
    # nothing sets the flag: the wait gives up after its limit and says so
    assert lib.amemDeviceWaitProbe(300, 0, ctypes.byref(code), ctypes.byref(ms)) == 0
    assert code.value == 1, code.value                       # kDevBarrierTimeout
    assert 250.0 <= ms.value < 3000.0, ms.value
    # the context is alive: ordinary work still runs and is right
    a = torch.arange(1 << 20, device="cuda", dtype=torch.float32)
    assert float((a * 2).sum()) == float(2 * (a.double().sum()))
    from asystem_amem_b200.ops import gemm_bf16
    x = torch.ones(128, 64, device="cuda", dtype=torch.bfloat16)
    y = gemm_bf16(x, x)
    torch.cuda.synchronize()
    assert float(y[0, 0]) == 64.0
    # and a second probe behaves the same
    assert lib.amemDeviceWaitProbe(100, 0, ctypes.byref(code), ctypes.byref(ms)) == 0 and code.value == 1
    assert lib.amemDeviceWaitProbe(0, 0, None, None) != 0     # a limit is mandatory
