"""Pause / resume over the mock VMM backend: the plumbing configuration of the baseline
(world_size 2 over gloo, allreduce of 1,048,576 fp32 N(0,1) values seeded per rank, ten
pause/resume cycles, bitwise-equal results, no leaked allocations) plus scope, idempotence,
guard and split-communicator behaviour."""
import os

import numpy as np
import pytest

from mp_util import run_ranks


def _config1(rank, world, uid, port):
    import numpy as np
    import torch
    import torch.distributed as dist
    from asystem_amem_b200 import Communicator, backend_usage, mem_stats, pause_all, resume_all
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = Communicator.from_torch_distributed()
    g = torch.Generator().manual_seed(rank)  # "seed 0 per rank" stream: seed = rank
    x = torch.randn(1048576, generator=g, dtype=torch.float32)
    ref = x.clone()
    dist.all_reduce(ref)  # gloo's answer, for a tolerance check
    out0 = x.clone()
    comm.all_reduce(out0)
    close = bool(torch.allclose(out0, ref, rtol=1e-6, atol=1e-6))
    base = backend_usage()
    st0 = mem_stats()
    bitwise = True
    freed = []
    for cycle in range(10):
        pause_all()
        during = backend_usage()
        freed.append(base["physical_bytes"] - during["physical_bytes"])
        assert during["mappings"] == 0, during
        resume_all()
        y = x.clone()
        comm.all_reduce(y)
        bitwise = bitwise and bool(torch.equal(y, out0))
    after = backend_usage()
    st1 = mem_stats()
    comm.destroy()
    end = backend_usage()
    dist.destroy_process_group()
    return {
        "close": close, "bitwise": bitwise, "freed": freed,
        "leak_bytes": after["physical_bytes"] - base["physical_bytes"],
        "leak_maps": after["mappings"] - base["mappings"],
        "end_bytes": end["physical_bytes"], "end_maps": end["mappings"],
        "pauses": st1["pause_count"] - st0["pause_count"],
        "live": st1["live_bytes"], "paused_bytes": st1["paused_bytes"],
    }


def test_config1_gloo_world2_ten_cycles():
    port = 29000 + os.getpid() % 2000
    res = run_ranks(_config1, 2, args=(port,), timeout=300, env={"AMEM_PAUSE_CONTROL": "1"})
    for r in res:
        assert r["close"] and r["bitwise"], r
        assert r["leak_bytes"] == 0 and r["leak_maps"] == 0, r
        assert r["end_bytes"] == 0 and r["end_maps"] == 0, r
        assert all(f > 0 and f == r["freed"][0] for f in r["freed"]), r
        assert r["pauses"] == 10 and r["paused_bytes"] == 0, r


def _scope_and_guard(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError, backend_usage, mem_alloc, mem_free, pause_all, resume_all
    import ctypes
    comm = Communicator(world, rank, uid)
    out = {}
    x = np.arange(1000, dtype=np.float32) + rank
    exp = sum(np.arange(1000, dtype=np.float32) + r for r in range(world))
    # user allocation: contents must survive a process-wide pause at the same address
    p = mem_alloc(1 << 16)
    buf = (ctypes.c_uint8 * (1 << 16)).from_address(p)
    for i in range(0, 1 << 16, 997):
        buf[i] = (i * 7 + rank) & 0xFF
    # communicator-scoped pause is idempotent and guards collectives
    comm.pause()
    comm.pause()
    try:
        comm.all_reduce(x.copy())
        out["guard"] = False
    except NcclError as e:
        out["guard"] = e.code == 5
    comm.resume()
    comm.resume()
    y = x.copy()
    comm.all_reduce(y)
    out["after_scoped"] = bool(np.array_equal(y, exp))
    pause_all()
    out["nothing_mapped"] = backend_usage()["mappings"] == 0
    try:
        mem_alloc(4096)
        out["alloc_refused"] = False
    except NcclError as e:
        out["alloc_refused"] = e.code == 5
    resume_all()
    out["user_contents"] = all(buf[i] == ((i * 7 + rank) & 0xFF) for i in range(0, 1 << 16, 997))
    y = x.copy()
    comm.all_reduce(y)
    out["after_all"] = bool(np.array_equal(y, exp))
    st = comm.pause_resume_stats()
    out["stateful_only"] = 0 < st["bytes_offloaded"] < st["bytes_released_local"]
    mem_free(p)
    comm.destroy()
    out["clean"] = backend_usage()["physical_bytes"] == 0
    return out


def test_scope_guard_and_user_memory():
    for r in run_ranks(_scope_and_guard, 2, env={"AMEM_PAUSE_CONTROL": "1"}):
        assert all(r.values()), r


def _split_hybrid(rank, world, uid, cycles):
    """TP=2 x EP/DP=world/2 split communicators, all paused and resumed together."""
    import numpy as np
    from asystem_amem_b200 import Communicator, backend_usage, pause_all, resume_all
    comm = Communicator(world, rank, uid)
    tp = comm.split(rank // 2, rank)      # pairs
    ep = comm.split(rank % 2, rank)       # strided groups
    none = comm.split(-1 if rank else 0, 0)
    ok = (tp.nranks == 2 and ep.nranks == world // 2 and (none is None) == (rank != 0))
    x = np.full(4096, float(rank + 1), dtype=np.float32)
    def run():
        a, b, c = x.copy(), x.copy(), x.copy()
        comm.all_reduce(a)
        tp.all_reduce(b)
        ep.all_reduce(c)
        return a, b, c
    first = run()
    exp_world = sum(range(1, world + 1))
    base = (rank // 2) * 2
    exp_tp = (base + 1) + (base + 2)
    exp_ep = sum(r + 1 for r in range(world) if r % 2 == rank % 2)
    ok = ok and first[0][0] == exp_world and first[1][0] == exp_tp and first[2][0] == exp_ep
    usage0 = backend_usage()["physical_bytes"]
    for _ in range(cycles):
        pause_all()
        assert backend_usage()["mappings"] == 0
        resume_all()
        again = run()
        ok = ok and all(np.array_equal(p, q) for p, q in zip(first, again))
    ok = ok and backend_usage()["physical_bytes"] == usage0
    for c in (none, ep, tp, comm):
        if c is not None:
            c.destroy()
    return bool(ok)


def test_split_communicators_pause_together():
    assert all(run_ranks(_split_hybrid, 4, args=(5,), env={"AMEM_STAGE_MB": "8", "AMEM_PAUSE_CONTROL": "1"}))


def _resident_control(rank, world, uid):
    """Default mode: the 2 MiB control segment stays mapped through a pause, only staging goes."""
    import numpy as np
    from asystem_amem_b200 import Communicator, backend_usage, pause_all, resume_all
    comm = Communicator(world, rank, uid)
    x = np.arange(4096, dtype=np.float32) * (rank + 1)
    first = x.copy()
    comm.all_reduce(first)
    before = backend_usage()
    ok = True
    for _ in range(3):
        pause_all()
        during = backend_usage()
        ok = ok and during["mappings"] == world            # my control block and the peers'
        ok = ok and 0 < during["physical_bytes"] < before["physical_bytes"]
        resume_all()
        y = x.copy()
        comm.all_reduce(y)
        ok = ok and bool(np.array_equal(y, first))
    st = comm.pause_resume_stats()
    ok = ok and st["bytes_offloaded"] == 0 and st["n_release_peer"] == world - 1
    ok = ok and backend_usage() == before
    comm.destroy()
    return bool(ok)


def test_control_segment_stays_resident_by_default():
    assert all(run_ranks(_resident_control, 3))


def test_random_alloc_free_pause_resume_sequence_keeps_contents_and_leaks_nothing():
    """Process-level scope (ncclMemAlloc memory, no communicator): a seeded random walk of
    allocate / free / pause / resume; every live buffer keeps its address and contents across
    every pause, allocations are refused while paused, nothing is left mapped at the end."""
    import ctypes
    import random
    os.environ["AMEM_BACKEND"] = "mock"
    from asystem_amem_b200 import NcclError, backend_usage, mem_alloc, mem_free, mem_stats, pause_all, resume_all
    rnd = random.Random(2024)
    base = backend_usage()["physical_bytes"]
    live = {}                                    # ptr -> (size, seed)
    paused = False

    def fill(ptr, size, seed):
        buf = (ctypes.c_uint8 * size).from_address(ptr)
        for i in range(0, size, 4093):
            buf[i] = (i * 31 + seed) & 0xFF

    def intact(ptr, size, seed):
        buf = (ctypes.c_uint8 * size).from_address(ptr)
        return all(buf[i] == ((i * 31 + seed) & 0xFF) for i in range(0, size, 4093))

    pauses = 0
    for step in range(200):
        action = rnd.choice(["alloc", "alloc", "free", "pause", "resume"])
        if action == "alloc":
            size = rnd.choice([1, 4096, 70_000, 1 << 20, 3 << 20])
            if paused:
                with pytest.raises(NcclError):
                    mem_alloc(size)
            elif len(live) < 24:
                p = mem_alloc(size)
                assert p not in live
                live[p] = (size, step)
                fill(p, size, step)
        elif action == "free" and live and not paused:
            p = rnd.choice(sorted(live))
            size, seed = live.pop(p)
            assert intact(p, size, seed)
            mem_free(p)
        elif action == "pause" and not paused:
            pause_all()
            paused = True
            pauses += 1
            assert backend_usage()["physical_bytes"] == base, "a pause must return every physical byte"
        elif action == "resume" and paused:
            resume_all()
            paused = False
            assert all(intact(p, s, seed) for p, (s, seed) in live.items())
    if paused:
        resume_all()
    assert pauses > 10 and all(intact(p, s, seed) for p, (s, seed) in live.items())
    for p in sorted(live):
        mem_free(p)
    assert backend_usage()["physical_bytes"] == base
    assert mem_stats()["live_bytes"] == 0 or backend_usage()["physical_bytes"] == base


def _two_groups(rank, world, _uid, share_dir):
    """Two co-located process groups with their own group ids (the reference's AMEM_GROUPID /
    ncclSetGroupID): socket names do not collide, and one group pauses while the other works."""
    import time
    import numpy as np
    from asystem_amem_b200 import Communicator, backend_usage, get_unique_id, mem_stats, set_group_id
    group, local = rank // 2, rank % 2
    set_group_id(group + 1)                          # before anything is allocated
    path = os.path.join(share_dir, f"uid_{group}")
    if local == 0:
        uid = get_unique_id()
        with open(path + ".tmp", "wb") as f:
            f.write(uid)
        os.rename(path + ".tmp", path)
    else:
        for _ in range(400):
            if os.path.exists(path):
                break
            time.sleep(0.05)
        uid = open(path, "rb").read()
    comm = Communicator(2, local, uid)
    out = {"gid": mem_stats()["group_id"] == group + 1}
    x = np.full(1000, float(local + 1 + 10 * group), dtype=np.float32)
    comm.all_reduce(x)
    out["first"] = bool(np.all(x == 3.0 + 20 * group))
    held = backend_usage()["physical_bytes"]
    for cycle in range(3):
        if group == cycle % 2:                       # the groups take turns being parked
            comm.pause()
            out[f"released {cycle}"] = backend_usage()["physical_bytes"] < held
            comm.resume()
        y = np.full(1000, float(local + 1), dtype=np.float32)
        comm.all_reduce(y)
        out[f"sum {cycle}"] = bool(np.all(y == 3.0))
    comm.destroy()
    return out


def test_two_process_groups_with_their_own_group_ids(tmp_path):
    for r in run_ranks(_two_groups, 4, args=(str(tmp_path),), timeout=300):
        assert all(r.values()), r
