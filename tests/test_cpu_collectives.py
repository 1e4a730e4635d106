"""CPU tests of the collective protocol over the mock VMM backend (2-4 rank processes)."""
import numpy as np
import pytest

from mp_util import run_ranks


def _all_collectives(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator
    comm = Communicator(world, rank, uid)
    rng = np.random.default_rng(1234)
    data = [rng.standard_normal(10007).astype(np.float32) for _ in range(world)]
    out = {}
    # all-reduce sum (one-shot size), then a large one that needs several chunks (two-shot)
    x = data[rank].copy()
    comm.all_reduce(x)
    ref = data[0].copy()
    for r in range(1, world):
        ref = ref + data[r]
    out["ar_small"] = bool(np.array_equal(x, ref))
    big = [np.random.default_rng(r).standard_normal(1 << 20).astype(np.float32) for r in range(world)]
    y = big[rank].copy()
    comm.all_reduce(y)
    # two-shot reduces slice by slice in rank order 0..n-1, same as this reference
    ref = big[0].copy()
    for r in range(1, world):
        ref = ref + big[r]
    out["ar_big"] = bool(np.array_equal(y, ref))
    # max on int32
    xi = (np.arange(1000, dtype=np.int32) * (rank + 1)) % 977
    exp = np.max(np.stack([(np.arange(1000, dtype=np.int32) * (r + 1)) % 977 for r in range(world)]), axis=0)
    comm.all_reduce(xi, op="max")
    out["ar_max"] = bool(np.array_equal(xi, exp))
    # all-gather
    g = np.empty(world * 5001, dtype=np.float32)
    comm.all_gather(data[rank][:5001].copy(), g)
    out["ag"] = bool(np.array_equal(g, np.concatenate([d[:5001] for d in data])))
    # reduce-scatter
    n = 3000
    send = np.stack([data[rank][:n] * (j + 1) for j in range(world)]).reshape(-1).copy()
    recv = np.empty(n, dtype=np.float32)
    comm.reduce_scatter(send, recv)
    ref = data[0][:n] * (rank + 1)
    for r in range(1, world):
        ref = ref + data[r][:n] * (rank + 1)
    out["rs"] = bool(np.array_equal(recv, ref))
    # broadcast from the last rank, reduce to rank 0
    b = data[rank][:777].copy()
    comm.broadcast(b, root=world - 1)
    out["bcast"] = bool(np.array_equal(b, data[world - 1][:777]))
    rd = np.empty(4099, dtype=np.float32)
    comm.reduce(data[rank][:4099].copy(), rd, root=0)
    if rank == 0:
        ref = data[0][:4099].copy()
        for r in range(1, world):
            ref = ref + data[r][:4099]
        out["reduce"] = bool(np.array_equal(rd, ref))
    # all-to-all
    s = np.concatenate([np.full(123, rank * 100 + j, dtype=np.int64) for j in range(world)])
    t = np.empty_like(s)
    comm.all_to_all(s, t)
    out["a2a"] = bool(np.array_equal(t, np.concatenate([np.full(123, j * 100 + rank, dtype=np.int64) for j in range(world)])))
    comm.destroy()
    return out


@pytest.mark.parametrize("world", [2, 4])
def test_collectives_match_numpy(world):
    res = run_ranks(_all_collectives, world)
    for r, d in enumerate(res):
        bad = [k for k, v in d.items() if not v]
        assert not bad, f"rank {r}: mismatch in {bad}"


def _flag_in_data_alltoall(rank, world, uid):
    """The opt-in small-message all-to-all (8-byte packets that carry their own flag): odd byte
    counts, repeated operations (slots alternate and are reused after the receiver's ack), a
    pause in between (fresh staging memory must not look like packets)."""
    import numpy as np
    from asystem_amem_b200 import Communicator
    comm = Communicator(world, rank, uid)
    ok = True
    for it, n in enumerate([1, 3, 7, 250, 1001, 250, 1, 1777, 64, 5]):
        send = np.concatenate([np.full(n, 16 * rank + q + it, dtype=np.uint8) for q in range(world)])
        recv = np.zeros_like(send)
        comm.all_to_all(send, recv)
        exp = np.concatenate([np.full(n, 16 * q + rank + it, dtype=np.uint8) for q in range(world)])
        ok = ok and bool(np.array_equal(recv, exp))
        if it == 4:
            comm.pause()
            comm.resume()
    comm.destroy()
    return ok


def test_flag_in_data_alltoall():
    assert all(run_ranks(_flag_in_data_alltoall, 4, env={"AMEM_LL": "1"}))


def _sendrecv_ring(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator, group_end, group_start
    comm = Communicator(world, rank, uid)
    ok = True
    for n in (1, 1000, 300000):  # the last one needs several credit rounds per lane
        send = np.full(n, rank + 1, dtype=np.float32)
        recv = np.zeros(n, dtype=np.float32)
        group_start()
        comm.send(send, (rank + 1) % world)
        comm.recv(recv, (rank - 1) % world)
        group_end()
        ok = ok and bool(np.all(recv == ((rank - 1) % world) + 1))
    comm.destroy()
    return ok


def test_sendrecv_ring():
    assert all(run_ranks(_sendrecv_ring, 3))


def _big_group(rank, world, uid):
    """More point-to-point operations in one group than one launch carries (a pipeline stage that
    also does an all-to-all-v): several messages per peer and direction, 24 operations in all."""
    import numpy as np
    from asystem_amem_b200 import Communicator, group_end, group_start
    comm = Communicator(world, rank, uid)
    per_peer = 4
    sends, recvs = {}, {}
    group_start()
    for q in range(world):
        if q == rank:
            continue
        for j in range(per_peer):
            n = 100 + 5000 * j
            sends[(q, j)] = np.full(n, 1000 * rank + 10 * q + j, dtype=np.float32)
            recvs[(q, j)] = np.zeros(n, dtype=np.float32)
            comm.send(sends[(q, j)], q)
            comm.recv(recvs[(q, j)], q)
    group_end()
    ok = all(bool(np.all(buf == 1000 * q + 10 * rank + j)) for (q, j), buf in recvs.items())
    comm.destroy()
    return ok and len(recvs) == per_peer * (world - 1)


def test_group_with_more_operations_than_one_launch_carries():
    assert all(run_ranks(_big_group, 4))


def _multi_chunk(rank, world, uid):
    """Messages several times larger than a staging slot: the chunked credit protocol."""
    import numpy as np
    from asystem_amem_b200 import Communicator
    comm = Communicator(world, rank, uid)
    n = 700_001                      # ~2.7 MiB of fp32 per rank, slots are 256 KiB here
    mine = (np.arange(n, dtype=np.float32) % 1013) + 7 * rank
    out = {}
    g = np.empty(world * n, dtype=np.float32)
    comm.all_gather(mine, g)
    out["ag"] = bool(np.array_equal(g, np.concatenate([(np.arange(n, dtype=np.float32) % 1013) + 7 * r for r in range(world)])))
    send = np.concatenate([mine + j for j in range(world)])
    recv = np.empty(n, dtype=np.float32)
    comm.reduce_scatter(send, recv)
    exp = sum(((np.arange(n, dtype=np.float32) % 1013) + 7 * r + rank) for r in range(world))
    out["rs"] = bool(np.array_equal(recv, exp))
    t = np.empty(world * n, dtype=np.float32)
    comm.all_to_all(send, t)
    out["a2a"] = bool(np.array_equal(t, np.concatenate([(np.arange(n, dtype=np.float32) % 1013) + 7 * j + rank for j in range(world)])))
    # and a small operation right after, on the barrier protocol
    x = np.ones(100, dtype=np.float32)
    comm.all_reduce(x)
    out["ar_after"] = bool(np.all(x == world))
    comm.destroy()
    return out


def test_multi_chunk_collectives():
    for d in run_ranks(_multi_chunk, 3, env={"AMEM_STAGE_MB": "7", "AMEM_P2P_SLOT_KB": "4"}):
        assert all(d.values()), d


def _alltoallv(rank, world, uid):
    import numpy as np
    from asystem_amem_b200 import Communicator
    comm = Communicator(world, rank, uid)
    # rank i sends (i + 2 * j + 1) * 1000 + 3 elements to rank j, except nothing from 0 to 1
    cnt = lambda i, j: 0 if (i, j) == (0, 1) else (i + 2 * j + 1) * 1000 + 3  # noqa: E731
    sc = [cnt(rank, j) for j in range(world)]
    rc = [cnt(j, rank) for j in range(world)]
    send = np.concatenate([np.full(sc[j], 100.0 * rank + j, dtype=np.float32) for j in range(world)])
    recv = np.full(sum(rc), -1.0, dtype=np.float32)
    ok = True
    for _ in range(2):
        comm.all_to_all_v(send, recv, sc, rc)
        exp = np.concatenate([np.full(rc[j], 100.0 * j + rank, dtype=np.float32) for j in range(world)])
        ok = ok and bool(np.array_equal(recv, exp))
        recv[:] = -1.0
    comm.destroy()
    return ok


def test_all_to_all_v():
    assert all(run_ranks(_alltoallv, 3))


def _fuzz(rank, world, uid, seed, cases):
    """Random (collective, type, operator, size) cases against numpy, same order of additions
    (rank 0 .. n-1), so floating-point results must match bit for bit.  Sizes run from one
    element to several staging slots so that single-chunk, multi-chunk and ragged-tail paths of
    every body are hit; the staging guard (AMEM_CANARY) is checked at the end."""
    import numpy as np
    from asystem_amem_b200 import Communicator
    comm = Communicator(world, rank, uid)
    rng = np.random.default_rng(seed)              # same stream on every rank: same cases
    dtypes = [np.float32, np.float64, np.int32, np.int64, np.uint8]
    bad = []

    def make(r, n, dt, salt):
        g = np.random.default_rng(1000 * salt + r)
        if np.issubdtype(dt, np.floating):
            return g.standard_normal(n).astype(dt)
        return g.integers(0, 7, n).astype(dt)

    def fold(arrs, op):
        acc = arrs[0].copy()
        for a in arrs[1:]:
            acc = {"sum": acc + a, "max": np.maximum(acc, a), "min": np.minimum(acc, a), "prod": acc * a}[op]
        return acc.astype(arrs[0].dtype)

    for case in range(cases):
        kind = ["allreduce", "allgather", "reducescatter", "alltoall", "broadcast", "reduce"][int(rng.integers(0, 6))]
        dt = dtypes[int(rng.integers(0, len(dtypes)))]
        op = ["sum", "max", "min", "prod"][int(rng.integers(0, 4))]
        n = int(rng.choice([1, 2, 3, 17, 255, 4097, 65537, int(rng.integers(1, 900_000))]))
        root = int(rng.integers(0, world))
        ok = True
        if kind == "allreduce":
            xs = [make(r, n, dt, case) for r in range(world)]
            x = xs[rank].copy()
            comm.all_reduce(x, op=op)
            ok = np.array_equal(x, fold(xs, op))
        elif kind == "allgather":
            xs = [make(r, n, dt, case) for r in range(world)]
            out = np.empty(world * n, dtype=dt)
            comm.all_gather(xs[rank].copy(), out)
            ok = np.array_equal(out, np.concatenate(xs))
        elif kind == "reducescatter":
            xs = [make(r, world * n, dt, case) for r in range(world)]
            out = np.empty(n, dtype=dt)
            comm.reduce_scatter(xs[rank].copy(), out, op=op)
            ok = np.array_equal(out, fold([x[rank * n:(rank + 1) * n] for x in xs], op))
        elif kind == "alltoall":
            xs = [make(r, world * n, dt, case) for r in range(world)]
            out = np.empty(world * n, dtype=dt)
            comm.all_to_all(xs[rank].copy(), out)
            ok = np.array_equal(out, np.concatenate([xs[j][rank * n:(rank + 1) * n] for j in range(world)]))
        elif kind == "broadcast":
            xs = [make(r, n, dt, case) for r in range(world)]
            x = xs[rank].copy()
            comm.broadcast(x, root=root)
            ok = np.array_equal(x, xs[root])
        else:
            xs = [make(r, n, dt, case) for r in range(world)]
            out = np.zeros(n, dtype=dt)
            comm.reduce(xs[rank].copy(), out, root=root, op=op)
            ok = rank != root or np.array_equal(out, fold(xs, op))
        if not ok:
            bad.append((case, kind, np.dtype(dt).name, op, n, root))
    comm.check_canary()
    comm.destroy()
    return bad


@pytest.mark.parametrize("world,seed", [(2, 11), (3, 12)])
def test_random_cases_match_numpy_bit_for_bit(world, seed):
    # a small staging segment makes most of the random sizes span several chunks
    for bad in run_ranks(_fuzz, world, args=(seed, 200), timeout=600, env={"AMEM_STAGE_MB": "8", "AMEM_CANARY": "1"}):
        assert bad == [], bad


def _fp8(rank, world, uid):
    import torch
    from asystem_amem_b200 import Communicator, NcclError
    comm = Communicator(world, rank, uid)
    out = {}
    for dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        n = 70_001
        mine = (torch.arange(n) % 13 + rank).float().to(dt)
        every = [(torch.arange(n) % 13 + r).float().to(dt) for r in range(world)]
        g = torch.empty(world * n, dtype=dt)
        comm.all_gather(mine, g)
        out[f"ag {dt}"] = bool(torch.equal(g.view(torch.uint8), torch.cat(every).view(torch.uint8)))
        b = mine.clone()
        comm.broadcast(b, root=world - 1)
        out[f"bcast {dt}"] = bool(torch.equal(b.view(torch.uint8), every[world - 1].view(torch.uint8)))
        send = torch.cat([(torch.full((500,), float(rank + j))).to(dt) for j in range(world)])
        recv = torch.empty_like(send)
        comm.all_to_all(send, recv)
        exp = torch.cat([(torch.full((500,), float(j + rank))).to(dt) for j in range(world)])
        out[f"a2a {dt}"] = bool(torch.equal(recv.view(torch.uint8), exp.view(torch.uint8)))
        try:
            comm.all_reduce(mine.clone())
            out[f"reduce refused {dt}"] = False
        except NcclError as e:
            out[f"reduce refused {dt}"] = e.code == 4
    comm.destroy()
    return out


def test_8bit_floats_ride_the_copy_collectives():
    for r in run_ranks(_fp8, 2):
        assert all(r.values()), r
