"""C API surface through ctypes on the mock backend: version / error strings, group ids,
ncclCommInitAll with in-process ranks, pre-multiplied-sum operators, unsupported calls,
memory statistics by category."""
import ctypes
import os
import threading

import numpy as np
import pytest

from mp_util import run_ranks


def _api(rank, world, uid):
    import ctypes
    import numpy as np
    from asystem_amem_b200 import Communicator, bindings as B, get_group_id, mem_stats
    lib = B.load_library()
    out = {}
    v = ctypes.c_int()
    lib.ncclGetVersion(ctypes.byref(v))
    out["version"] = v.value == 22705
    out["errstr"] = lib.ncclGetErrorString(5) == b"invalid usage"
    out["group_env"] = get_group_id() == 170           # AMEM_GROUPID from the environment
    comm = Communicator(world, rank, uid)
    out["group_locked"] = lib.ncclSetGroupID(7) != 0   # too late: memory is already tracked
    # pre-multiplied sum
    lib.ncclRedOpCreatePreMulSum.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    op = ctypes.c_int()
    scalar = ctypes.c_float(0.5)
    assert lib.ncclRedOpCreatePreMulSum(ctypes.byref(op), ctypes.byref(scalar), B.DTYPES["float32"], 1, comm._h) == 0
    x = np.full(1000, float(rank + 1), dtype=np.float32)
    assert lib.ncclAllReduce(x.ctypes.data, x.ctypes.data, 1000, B.DTYPES["float32"], op.value, comm._h, None) == 0
    out["premul"] = bool(np.all(x == 0.5 * sum(range(1, world + 1))))
    lib.ncclRedOpDestroy.argtypes = [ctypes.c_int, ctypes.c_void_p]
    assert lib.ncclRedOpDestroy(op.value, comm._h) == 0
    out["destroyed_op_refused"] = lib.ncclAllReduce(x.ctypes.data, x.ctypes.data, 1000, B.DTYPES["float32"], op.value, comm._h, None) == 4
    # a shrink that names the caller itself, or a rank that does not exist, is refused
    lib.ncclCommShrink.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_int]
    nc = ctypes.c_void_p()
    me, bogus = (ctypes.c_int * 1)(rank), (ctypes.c_int * 1)(world + 5)
    out["shrink"] = (lib.ncclCommShrink(comm._h, me, 1, ctypes.byref(nc), None, 0) == 4 and
                     lib.ncclCommShrink(comm._h, bogus, 1, ctypes.byref(nc), None, 0) == 4 and not nc.value)
    st = mem_stats()
    out["stats"] = (st["n_local"] == 2 and st["n_imported"] == 2 * (world - 1) and st["scratch_bytes"] > st["stateful_bytes"] > 0
                    and st["bytes_by_tag"][1] > 0 and st["bytes_by_tag"][7] > 0 and st["group_id"] == 170)
    # a simulated group: nothing is sent, the estimate is positive, the next real group works
    class SimInfo(ctypes.Structure):
        _fields_ = [("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint), ("estimatedTime", ctypes.c_float)]
    sim = SimInfo(ctypes.sizeof(SimInfo), 0x74685283, 22705, -1.0)
    buf = np.zeros(1 << 16, dtype=np.float32)
    lib.ncclGroupStart()
    lib.ncclSend(buf.ctypes.data, buf.size, B.DTYPES["float32"], (rank + 1) % world, comm._h, None)
    lib.ncclRecv(buf.ctypes.data, buf.size, B.DTYPES["float32"], (rank - 1) % world, comm._h, None)
    lib.ncclGroupSimulateEnd.argtypes = [ctypes.POINTER(SimInfo)]
    out["simulate"] = lib.ncclGroupSimulateEnd(ctypes.byref(sim)) == 0 and sim.estimatedTime > 0
    out["simulate_bad_struct"] = lib.ncclGroupSimulateEnd(ctypes.byref(SimInfo(1, 2, 3, 0.0))) == 4
    y = np.full(10, float(rank), dtype=np.float32)
    assert lib.ncclAllReduce(y.ctypes.data, y.ctypes.data, 10, B.DTYPES["float32"], 0, comm._h, None) == 0
    out["after_simulate"] = bool(np.all(y == sum(range(world))))
    lib.ncclResetDebugInit()
    bad = np.zeros(4, dtype=np.float32)
    out["bad_root"] = lib.ncclBroadcast(bad.ctypes.data, bad.ctypes.data, 4, B.DTYPES["float32"], world + 3, comm._h, None) == 4
    comm.destroy()
    return out


def test_c_api_surface():
    for r in run_ranks(_api, 2, env={"AMEM_GROUPID": "170"}):
        assert all(r.values()), r


def test_comm_init_all_in_one_process():
    os.environ["AMEM_BACKEND"] = "mock"
    from asystem_amem_b200 import bindings as B
    lib = B.load_library()
    n = 3
    comms = (ctypes.c_void_p * n)()
    lib.ncclCommInitAll.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p]
    assert lib.ncclCommInitAll(comms, n, None) == 0
    bufs = [np.full(5000, float(i + 1), dtype=np.float32) for i in range(n)]

    def run(i):
        assert lib.ncclAllReduce(bufs[i].ctypes.data, bufs[i].ctypes.data, 5000, B.DTYPES["float32"], 0, comms[i], None) == 0

    th = [threading.Thread(target=run, args=(i,)) for i in range(n)]
    [t.start() for t in th]
    [t.join(60) for t in th]
    assert all(np.all(b == 6.0) for b in bufs)
    # process-wide pause with several ranks of one communicator in this process
    assert lib.ncclPause(None) == 0
    assert lib.ncclAllReduce(bufs[0].ctypes.data, bufs[0].ctypes.data, 5000, B.DTYPES["float32"], 0, comms[0], None) == 5
    assert lib.ncclResume(None) == 0
    th = [threading.Thread(target=run, args=(i,)) for i in range(n)]
    [t.start() for t in th]
    [t.join(60) for t in th]
    assert all(np.all(b == 18.0) for b in bufs)
    th = [threading.Thread(target=lambda i=i: lib.ncclCommDestroy(comms[i])) for i in range(n)]
    [t.start() for t in th]
    [t.join(60) for t in th]


def test_gemm_planner_picks_tile_form_and_tail_split():
    """The GEMM's tiling is host arithmetic: checked here for the shapes it was calibrated on
    (148 SMs), without a GPU."""
    os.environ["AMEM_BACKEND"] = "mock"
    from asystem_amem_b200 import bindings as B
    lib = B.load_library()

    def plan(M, N, K, **env):
        old = {k: os.environ.get(k) for k in env}
        os.environ.update({k: str(v) for k, v in env.items()})
        try:
            r, c, s = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
            assert lib.amemGemmPlan(M, N, K, 148, ctypes.byref(r), ctypes.byref(c), ctypes.byref(s)) == 0
            return r.value, c.value, s.value
        finally:
            for k, v in old.items():
                os.environ.pop(k, None) if v is None else os.environ.__setitem__(k, v)

    # tensor-parallel MLP shape: 256-row tiles, 448 tiles = 3 waves + 4 tiles cut into K-slices
    rows, cols, slices = plan(8192, 3584, 8192)
    assert (rows, cols) == (256, 256) and 4 <= slices <= 32
    # forced 128-row tiles: 896 tiles = 6 waves + 8 tiles; min(148 // 8, 128 K blocks // 8) = 16 slices
    assert plan(8192, 3584, 8192, AMEM_GEMM_TALL=0) == (128, 256, 16)
    assert plan(8192, 3584, 8192, AMEM_GEMM_TALL=0, AMEM_GEMM_SPLITK=0)[2] == 1
    # short K or few tiles: the exposed epilogue of the tall form does not pay
    assert plan(2048, 2048, 2048)[0] == 128
    assert plan(1024, 3584, 8192)[0] == 128
    assert plan(64, 512, 4096)[0] == 128          # a single row block can never be tall
    # tile width stays a multiple of 32 in [128, 256]; bad shapes are refused
    for shape in [(4096, 4096, 4096), (1000, 264, 8192), (8192, 8192, 3584)]:
        rows, cols, slices = plan(*shape)
        assert rows in (128, 256) and 128 <= cols <= 256 and cols % 32 == 0 and 1 <= slices <= 32
    assert lib.amemGemmPlan(128, 100, 64, 148, None, None, None) == 4   # N not a multiple of 8


def test_all_gather_gemm_plan_picks_schedule_and_flag_granularity(monkeypatch):
    """Mover warps inside every CTA up to four ranks, dedicated mover CTAs from five up (an
    environment variable forces either); a ready flag covers as few rows as the flag array and the
    movers' smallest copy allow, 32 rows on the mover-CTA schedule; shards too long for the flag
    array are refused."""
    import ctypes
    from asystem_amem_b200.bindings import load_library
    lib = load_library()
    w, per, flags = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()

    def plan(n, rows, K):
        rc = lib.amemAllGatherGemmPlan(n, rows, K, ctypes.byref(w), ctypes.byref(per), ctypes.byref(flags))
        return rc, w.value, per.value, flags.value

    monkeypatch.delenv("AMEM_AG_DESIGN", raising=False)
    assert plan(2, 4096, 8192) == (0, 1, 4, 1024)          # 1024 flags at most: 4 rows each
    assert plan(4, 2048, 8192) == (0, 1, 2, 1024)
    assert plan(4, 1024, 8192) == (0, 1, 1, 1024)          # one 16 KB row is more than the smallest copy
    assert plan(4, 512, 256) == (0, 1, 16, 32)             # 512-byte rows: 16 of them make one 8 KB copy
    assert plan(8, 1024, 8192) == (0, 0, 32, 32)           # mover CTAs: a flag per 32 rows
    assert plan(5, 1000, 4096) == (0, 0, 32, 32)
    assert plan(8, 32 * 256 + 1, 4096)[0] != 0             # more than 256 flags on the mover-CTA schedule
    assert plan(4, 128, 100)[0] != 0                       # K not a multiple of 8
    monkeypatch.setenv("AMEM_AG_DESIGN", "1")
    assert plan(8, 1024, 8192)[:2] == (0, 1)
    monkeypatch.setenv("AMEM_AG_DESIGN", "2")
    assert plan(2, 1024, 8192)[:3] == (0, 0, 32)
    assert lib.amemAllGatherGemmPlan(4, 1024, 8192, None, None, None) == 0


def test_tuner_plan_is_deterministic_and_within_staging():
    """Variant picker: thresholds measured on 2 and 8 GPUs, chunk sizes that fit the staging
    layout, identical answers on repeated calls (every rank must pick the same plan)."""
    os.environ["AMEM_BACKEND"] = "mock"
    from asystem_amem_b200 import bindings as B
    lib = B.load_library()
    lib.amemTunerPlan.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                  ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_size_t)]
    BF16 = B.DTYPES["bfloat16"]

    def plan(kind, nbytes, n, nvls=1, dtype=BF16, es=2):
        a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()
        assert lib.amemTunerPlan(kind, nbytes // es, dtype, n, nvls, 0, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)) == 0
        return a.value, b.value, c.value * es

    ONE, TWO, NVLS = 1, 2, 3
    # all-reduce variants
    assert plan(0, 64 << 10, 8)[0] == ONE and plan(0, 256 << 10, 8)[0] == ONE
    assert plan(0, 1 << 20, 8)[0] == NVLS and plan(0, 1 << 30, 8)[0] == NVLS and plan(0, 1 << 30, 4)[0] == NVLS
    assert plan(0, 1 << 30, 8, nvls=0)[0] == TWO
    assert plan(0, 1 << 20, 2)[0] == ONE and plan(0, 16 << 20, 2)[0] == ONE     # two GPUs: one-shot up to 16 MiB
    assert plan(0, 32 << 20, 2)[0] == TWO and plan(0, 1 << 30, 2)[0] == TWO      # never NVLS between two GPUs
    # grid grows with the message and is capped
    assert plan(0, 8, 8)[1] == 1 and plan(0, 1 << 30, 8)[1] == 128
    # chunks: whole message up to 32 MiB (NVLS), then about eight chunks of at least 16 MiB, never above a third of a half
    stage = 288 << 20
    quarter = ((stage - 8 * 2 * 32 * (64 << 10)) // 4) & ~4095
    assert plan(0, 32 << 20, 8)[2] >= 32 << 20
    assert plan(0, 256 << 20, 8)[2] == 32 << 20
    assert 16 << 20 <= plan(0, 64 << 20, 8)[2] <= (2 * quarter) // 3
    assert plan(0, 8 << 30, 8)[2] <= (2 * quarter) // 3
    # all-gather / reduce-scatter / all-to-all: per-rank chunk never above one rank's slot of a quarter
    for kind in (1, 2, 5):
        for n in (2, 4, 8):
            for per_rank in (1 << 20, 40 << 20, 1 << 30):
                chunk = plan(kind, per_rank, n)[2]
                assert 0 < chunk <= max(per_rank, 4096) and chunk <= quarter // n + 4096
    # same question, same answer
    assert plan(0, 123456789 * 2, 8) == plan(0, 123456789 * 2, 8)
    assert lib.amemTunerPlan(9, 1, BF16, 8, 1, 0, None, None, None) == 4


def test_c_program_against_nccl_h_runs_pause_cycles(tmp_path):
    """examples/pause_cycle.c uses nothing but nccl.h (plus ncclPause / ncclResume / ncclMemStats):
    built with gcc against the in-tree library, three forked ranks on the mock backend."""
    import shutil
    import subprocess
    from asystem_amem_b200 import bindings as B
    B.load_library()
    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("gcc not available")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "asystem_amem_b200", "lib")
    exe = tmp_path / "pause_cycle"
    res = subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I" + os.path.join(root, "csrc", "include"),
                          os.path.join(root, "examples", "pause_cycle.c"), "-L" + libdir, "-lamem_b200",
                          "-Wl,-rpath," + libdir, "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    env = dict(os.environ, AMEM_BACKEND="mock", GMM_IPC_DIR=str(tmp_path), GMM_LOG="2")
    run = subprocess.run([str(exe), "3"], capture_output=True, text=True, timeout=300, env=env)
    assert run.returncode == 0 and "pause cycle ok: 3 ranks" in run.stdout, (run.stdout, run.stderr[-3000:])


def test_python_switch_example_runs_on_the_mock_backend():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, AMEM_BACKEND="mock", GMM_LOG="2")
    run = subprocess.run([sys.executable, os.path.join(root, "examples", "train_infer_switch.py"), "--cpu", "--cycles", "2"],
                         capture_output=True, text=True, timeout=300, env=env)
    assert run.returncode == 0 and "switch example ok" in run.stdout, (run.stdout, run.stderr[-3000:])


def test_timing_helpers_without_a_gpu():
    from asystem_amem_b200.utils.timing import ClockSampler, load_measured_peaks
    peaks = load_measured_peaks()
    assert peaks["hbm_gbs"] > 1000 and peaks["bf16_tflops"] > 100 and peaks["source"] in ("measured", "fallback")
    s = ClockSampler(0, period_s=None)          # no thread: samples only on request
    with s:
        s.sample_now()
    out = s.summary()
    assert set(out) == {"sm_mhz", "sm_max_mhz", "reasons", "samples"} and out["reasons"] == []


def test_json_log_lines_are_well_formed(tmp_path):
    """AMEM_LOG_JSON=1: every log line is one JSON object (level, pid, time, place, message)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from asystem_amem_b200 import Communicator, get_unique_id, mem_stats\n"
            "c = Communicator(1, 0, get_unique_id()); c.pause(); c.resume(); mem_stats(print_too=True); c.destroy()\n" % root)
    env = dict(os.environ, AMEM_BACKEND="mock", AMEM_LOG_JSON="1", GMM_LOG="5", GMM_IPC_DIR=str(tmp_path))
    run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, env=env)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stderr.splitlines() if l.startswith("{")]
    assert len(lines) >= 3
    for l in lines:
        rec = json.loads(l)
        assert rec["amem"] in ("FATAL", "ERROR", "WARN", "INFO", "DEBUG", "VERBOSE") and rec["pid"] > 0 and ":" in rec["at"] and "msg" in rec


def test_paused_context_manager():
    os.environ["AMEM_BACKEND"] = "mock"
    from asystem_amem_b200 import Communicator, NcclError, backend_usage, get_unique_id, paused
    c = Communicator(1, 0, get_unique_id())
    x = np.ones(10, dtype=np.float32)
    held = backend_usage()["physical_bytes"]
    with paused():                                   # whole process
        assert backend_usage()["physical_bytes"] < held
        with pytest.raises(NcclError):
            c.all_reduce(x)
    c.all_reduce(x)
    with pytest.raises(RuntimeError):
        with paused(c):                              # one communicator; resumed although the block raises
            raise RuntimeError("work failed while paused")
    assert backend_usage()["physical_bytes"] == held
    c.all_reduce(x)
    c.destroy()


def test_gemm_planner_invariants_on_random_shapes():
    import random
    os.environ["AMEM_BACKEND"] = "mock"
    from asystem_amem_b200 import bindings as B
    lib = B.load_library()
    rnd = random.Random(7)
    for _ in range(500):
        M, N, K = rnd.randint(1, 20000), 8 * rnd.randint(1, 2500), 8 * rnd.randint(1, 2500)
        sms = rnd.choice([1, 16, 132, 148, 160])
        r, c, s = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        assert lib.amemGemmPlan(M, N, K, sms, ctypes.byref(r), ctypes.byref(c), ctypes.byref(s)) == 0
        assert r.value in (128, 256) and (r.value == 128 or M > 128)
        assert 128 <= c.value <= 256 and c.value % 32 == 0
        assert 1 <= s.value <= 32
        k_blocks = (K + 63) // 64
        tiles = -(-M // r.value) * -(-N // c.value)
        if s.value > 1:                         # a split only of a partly filled last wave, in slices of >= 8 K blocks
            assert tiles % sms != 0 and s.value * (tiles % sms) <= sms and s.value <= max(1, k_blocks // 8)
