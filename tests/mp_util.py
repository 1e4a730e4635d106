"""Helpers to run a function as N CPU rank processes over the mock backend."""
import multiprocessing as mp
import os
import traceback


def _entry(fn, rank, world, uid, q, env, args):
    try:
        os.environ.update(env)
        res = fn(rank, world, uid, *args)
        q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def run_ranks(fn, world, args=(), env=None, timeout=120, expect_fail=False):
    """Spawns `world` processes running fn(rank, world, unique_id, *args) with the mock backend.
    Returns the list of per-rank results (or (status, payload) pairs when expect_fail)."""
    base_env = {"AMEM_BACKEND": "mock", "GMM_LOG": os.environ.get("GMM_LOG", "2")}
    base_env.update(env or {})
    saved = {k: os.environ.get(k) for k in base_env}
    os.environ.update(base_env)   # the unique id below is made under the same settings
    from asystem_amem_b200 import get_unique_id
    uid = get_unique_id()
    for k, v in saved.items():    # do not leak this test's settings into the next one
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, uid, q, base_env, args)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    import queue as _queue
    import time as _time
    deadline = _time.monotonic() + timeout
    try:
        while len(out) < world and _time.monotonic() < deadline:
            try:
                rank, status, payload = q.get(timeout=0.25)
                out[rank] = (status, payload)
            except _queue.Empty:
                # a rank that exited without reporting will never report
                if all((not p.is_alive()) for r, p in enumerate(procs) if r not in out):
                    try:
                        while True:
                            rank, status, payload = q.get(timeout=0.25)
                            out[rank] = (status, payload)
                    except _queue.Empty:
                        break
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    if expect_fail:
        return [out.get(r, ("missing", None)) for r in range(world)]
    for r in range(world):
        status, payload = out.get(r, ("missing", None))
        assert status == "ok", f"rank {r}: {payload}"
    return [out[r][1] for r in range(world)]
