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


def _fault_after_the_vote(rank, world, uid, what, nth, who):
    """A failure AFTER every rank agreed that its memory is back (handle export, descriptor
    passing, import, map): every rank must end PAUSED again, with nothing mapped, and a second
    ncclResume must succeed."""
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError, backend_usage, inject
    comm = Communicator(world, rank, uid)
    x = (np.arange(5000, dtype=np.float32) + rank)
    first = x.copy()
    comm.all_reduce(first)
    comm.pause()
    if rank == who:
        inject(what, nth)
    try:
        comm.resume()
        code = 0
    except NcclError as e:
        code = e.code
    rolled_back = backend_usage()["mappings"] == 0 and backend_usage()["physical_bytes"] == 0
    try:
        comm.all_reduce(x.copy())
        guarded = False
    except NcclError as e:
        guarded = e.code == 5
    comm.resume()  # nothing injected now
    again = x.copy()
    comm.all_reduce(again)
    comm.pause()   # and the communicator keeps cycling
    comm.resume()
    third = x.copy()
    comm.all_reduce(third)
    comm.destroy()
    return code, rolled_back, guarded, bool(np.array_equal(first, again) and np.array_equal(first, third))


# with two ranks and the control segment pausable, a resuming rank sends: its first vote, one handle
# per segment (2), its second vote ("nofd" counts only messages that carry a descriptor); and maps: its own two segments, then the peer's two
@pytest.mark.parametrize("what,nth,who", [("uds:drop", 2, 0), ("uds:nofd", 2, 0), ("vmm:export", 1, 0), ("vmm:import", 1, 1),
                                           ("vmm:import", 2, 1), ("vmm:map", 3, 1)])
def test_failure_after_the_resume_vote_rolls_back_and_resume_can_be_retried(what, nth, who):
    res = run_ranks(_fault_after_the_vote, 2, args=(what, nth, who), env=FAST)
    for code, rolled_back, guarded, same in res:
        assert code != 0 and rolled_back and guarded and same, res


def _pause_all_fault(rank, world, uid):
    """The same through ncclPause(NULL) / ncclResume(NULL) with two communicators and user memory:
    one pass serves all of them; after the failed pass everything is PAUSED, after the retry
    everything works."""
    import numpy as np
    from asystem_amem_b200 import Communicator, NcclError, inject, pause_all, resume_all
    comm = Communicator(world, rank, uid)
    sub = comm.split(0, rank)
    x = (np.arange(3000, dtype=np.float32) + rank)
    a = x.copy()
    comm.all_reduce(a)
    b = x.copy()
    sub.all_reduce(b)
    pause_all()
    if rank == 1:
        inject("vmm:import", 3)      # one of the second communicator's imports
    try:
        resume_all()
        code = 0
    except NcclError as e:
        code = e.code
    try:
        comm.all_reduce(x.copy())
        guarded = False
    except NcclError as e:
        guarded = e.code == 5
    resume_all()
    a2, b2 = x.copy(), x.copy()
    comm.all_reduce(a2)
    sub.all_reduce(b2)
    sub.destroy()
    comm.destroy()
    return code, guarded, bool(np.array_equal(a, a2) and np.array_equal(b, b2))


def test_process_wide_resume_failure_is_retried():
    res = run_ranks(_pause_all_fault, 2, env=FAST)
    for code, guarded, same in res:
        assert code != 0 and guarded and same, res


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
