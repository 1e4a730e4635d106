"""Failure detection and fault injection, host side only (mock backend, CPU rank processes).
Nothing here touches a GPU: failures are a rank that never joins or leaves between steps, a
dropped / truncated control message, a withheld file descriptor, an injected allocation
failure on resume, and a peer that never enters a collective (bounded wait runs out)."""
import os

import numpy as np
import pytest

from mp_util import run_ranks

FAST = {"AMEM_PAUSE_CONTROL": "1", "AMEM_OP_TIMEOUT_MS": "1500", "AMEM_INIT_TIMEOUT_MS": "1500", "AMEM_DEVICE_TIMEOUT_MS": "700", "GMM_LOG": "0"}


def _never_joins(rank, world, uid):
    from asystem_amem_b200 import Communicator, NcclError
    if rank == 1:
        return "absent"
    try:
        Communicator(world, rank, uid)
    except NcclError as e:
        return e.code
    return "no error"


def test_rank_never_joins_times_out():
    res = run_ranks(_never_joins, 2, env=FAST)
    assert res[0] == 2 and res[1] == "absent"  # ncclSystemError after the init deadline


def _rank_leaves(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError
    comm = Communicator(world, rank, uid)
    x = np.ones(100, dtype=np.float32)
    comm.all_reduce(x)
    if rank == 1:
        os._exit(0)  # leaves between steps without telling anybody
    try:
        comm.pause()
    except NcclError as e:
        return e.code
    return "no error"


def test_rank_leaves_between_steps_is_detected():
    res = run_ranks(_rank_leaves, 2, env=FAST, expect_fail=True)
    status, code = res[0]
    assert status == "ok" and code in (6, 2), res  # remote error (socket closed) or timeout


def _control_message_faults(rank, world, uid, kind):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError, inject
    comm = Communicator(world, rank, uid)
    x = np.ones(100, dtype=np.float32)
    comm.all_reduce(x)
    comm.pause()
    if rank == 0:
        inject("uds:" + kind, 1 if kind != "nofd" else 1)
    try:
        comm.resume()
        return "no error"
    except NcclError as e:
        return e.code


@pytest.mark.parametrize("kind,victim_codes", [("drop", (2, 6)), ("short", (6, 3, 2)), ("nofd", (2, 6))])
def test_control_plane_faults_surface_as_errors(kind, victim_codes):
    res = run_ranks(_control_message_faults, 2, args=(kind,), env=FAST, expect_fail=True)
    status, code = res[1]
    assert status == "ok" and code in victim_codes, res


def _oom_on_resume(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError, backend_usage, inject
    comm = Communicator(world, rank, uid)
    x = (np.arange(5000, dtype=np.float32) + rank)
    first = x.copy()
    comm.all_reduce(first)
    comm.pause()
    if rank == 1:
        inject("vmm:create", 2)  # second allocation of this resume fails
    codes = []
    try:
        comm.resume()
        codes.append(0)
    except NcclError as e:
        codes.append(e.code)
    rolled_back = backend_usage()["mappings"] == 0 and backend_usage()["physical_bytes"] == 0
    try:
        comm.all_reduce(x.copy())
        guarded = False
    except NcclError as e:
        guarded = e.code == 5
    comm.resume()  # nothing injected now
    again = x.copy()
    comm.all_reduce(again)
    comm.destroy()
    return codes[0], rolled_back, guarded, bool(np.array_equal(first, again))


def test_allocation_failure_on_resume_rolls_every_rank_back():
    res = run_ranks(_oom_on_resume, 2, env=FAST)
    assert res[1][0] == 1 and res[0][0] == 6, res      # failing rank: CUDA error, peer: remote error
    for code, rolled_back, guarded, same in res:
        assert rolled_back and guarded and same, res


def _peer_skips_collective(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError
    comm = Communicator(world, rank, uid)
    x = np.ones(10, dtype=np.float32)
    comm.all_reduce(x)
    if rank == 1:
        import time
        time.sleep(2.0)
        return "skipped"
    try:
        comm.all_reduce(x)
        first = 0
    except NcclError as e:
        first = e.code
    return first, comm.async_error()


def test_bounded_wait_runs_out_when_a_peer_skips_a_collective():
    res = run_ranks(_peer_skips_collective, 2, env=FAST)
    assert res[0] == (3, 3), res  # ncclInternalError, also visible through ncclCommGetAsyncError


def _shrink_after_loss(rank, world, uid):
    """Rank 2 leaves between steps (host-side failure, nothing in flight); the survivors build a
    smaller communicator out of the old one and carry on, pause / resume included."""
    import numpy as np
    from asystem_amem_b200 import Communicator
    comm = Communicator(world, rank, uid)
    x = np.full(1000, float(rank + 1), dtype=np.float32)
    comm.all_reduce(x)
    ok = bool(np.all(x == 6.0))
    if rank == 2:
        return ok                                     # gone: never calls shrink, never destroys
    small = comm.shrink([2])
    ok = ok and small.nranks == 2 and small.rank == rank
    y = np.full(1000, float(rank + 1), dtype=np.float32)
    small.all_reduce(y)
    ok = ok and bool(np.all(y == 3.0))
    small.pause()
    small.resume()
    y[:] = float(rank + 1)
    small.all_reduce(y)
    ok = ok and bool(np.all(y == 3.0))
    small.destroy()
    comm.abort()
    return ok


def test_survivors_shrink_the_communicator():
    assert all(run_ranks(_shrink_after_loss, 3, env=FAST))


def _guard_catches_overflow(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError
    comm = Communicator(world, rank, uid)
    x = np.ones(1 << 16, dtype=np.float32)
    comm.all_reduce(x)
    comm.check_canary()                      # clean after real traffic
    out = {"clean": True}
    if rank == 0:
        assert comm.lib.amemDebugDirtyCanary(comm._h) == 0
        try:
            comm.check_canary()
            out["caught"] = False
        except NcclError as e:
            out["caught"] = "guard is dirty" in str(e)
        try:
            comm.pause()                     # a dirty guard also refuses the pause
            out["pause_refused"] = False
        except NcclError:
            out["pause_refused"] = True
    comm.abort()
    return out


def test_staging_guard_reports_out_of_bounds_write():
    res = run_ranks(_guard_catches_overflow, 2, env=dict(FAST, AMEM_CANARY="1"))
    assert res[0] == {"clean": True, "caught": True, "pause_refused": True} and res[1] == {"clean": True}
