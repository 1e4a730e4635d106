"""Registered windows on CPU ranks (mock backend): memory from ncclMemAlloc that every rank maps,
used in place by the all-reduce, tracked by pause / resume like the communicator's own segments."""
import numpy as np

from mp_util import run_ranks

ENV = {"AMEM_PAUSE_CONTROL": "1", "GMM_LOG": "1"}


def _window_cycle(rank, world, uid):
    from asystem_amem_b200 import Communicator, NcclError, backend_usage, mem_stats, pause_all, resume_all
    comm = Communicator(world, rank, uid)
    n = 300_000                                   # 1.2 MB of fp32: above the window threshold
    win = comm.window_alloc(4 * n + 4096)
    x = win.tensor(np.float32, n)
    rng = np.random.default_rng(rank)
    mine = rng.standard_normal(n).astype(np.float32)
    expect = np.zeros(n, dtype=np.float32)
    for r in range(world):                        # the kernel adds in rank order 0..n-1
        expect = expect + np.random.default_rng(r).standard_normal(n).astype(np.float32)
    out = {}
    x[:] = mine
    comm.all_reduce(x, algo="window")             # in place, inside the window
    out["first"] = bool(np.array_equal(x, expect))
    stats = mem_stats()
    out["records"] = (stats["n_local"], stats["n_imported"])
    tail = win.tensor(np.uint8, 4096, offset_bytes=4 * n)
    tail[:] = rank + 7                            # user data in the window must survive a pause
    results = []
    for cycle in range(3):
        if cycle % 2 == 0:
            comm.pause()
        else:
            pause_all()
        out.setdefault("released", backend_usage()["physical_bytes"] == 0 and backend_usage()["mappings"] == 0)
        try:
            comm.all_reduce(x, algo="window")
            out["guard"] = False
        except NcclError as e:
            out.setdefault("guard", e.code == 5)
        if cycle % 2 == 0:
            comm.resume()
        else:
            resume_all()
        out["kept"] = out.get("kept", True) and bool(np.array_equal(x, expect)) and bool(np.all(tail == rank + 7))
        x[:] = mine
        comm.all_reduce(x)                        # the tuner picks the window path by itself
        results.append(bool(np.array_equal(x, expect)))
    out["after"] = all(results)
    # out of place, between two windows
    win2 = comm.window_alloc(4 * n)
    y = win2.tensor(np.float32, n)
    x[:] = mine
    comm.all_reduce(x, y, algo="window")
    out["out_of_place"] = bool(np.array_equal(y, expect)) and bool(np.array_equal(x, mine))
    win2.free()
    win.free()
    out["clean"] = mem_stats()["n_imported"] == stats["n_imported"] - (world - 1)
    comm.destroy()
    out["leak"] = backend_usage()["physical_bytes"] != 0
    return out


def _check(res, world):
    for out in res:
        assert out["first"] and out["after"] and out["kept"] and out["released"] and out["guard"] and out["out_of_place"], res
        assert out["clean"] and not out["leak"], res
        # control + staging + window on my side; the same three of every peer imported
        assert out["records"] == (3, 3 * (world - 1)), res


def test_window_allreduce_and_pause_two_ranks():
    _check(run_ranks(_window_cycle, 2, env=ENV), 2)


def test_window_allreduce_and_pause_four_ranks():
    _check(run_ranks(_window_cycle, 4, env=ENV), 4)


def _window_misuse(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError, mem_alloc, mem_free
    comm = Communicator(world, rank, uid)
    out = {}
    host = np.zeros(1024, dtype=np.float32)       # not from ncclMemAlloc
    try:
        comm.window_register(host.ctypes.data, host.nbytes)
        out["foreign"] = False
    except NcclError as e:
        out["foreign"] = e.code == 4
    p = mem_alloc(1 << 20)
    w = comm.window_register(p, 1 << 20)
    try:
        mem_free(p)                               # still registered
        out["free_refused"] = False
    except NcclError as e:
        out["free_refused"] = e.code == 5
    w.free()
    mem_free(p)
    comm.destroy()
    return out


def test_window_misuse_is_refused():
    for out in run_ranks(_window_misuse, 2, env=ENV):
        assert out == {"foreign": True, "free_refused": True}
