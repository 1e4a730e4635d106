"""Runs N ranks of one communicator as threads on cuda:0.  Ranks that share a process and a
GPU are emulated by the library as one cooperative grid, so the multi-rank kernels can be
checked on a single-GPU machine."""
import threading
import traceback

import torch


def run_emulated(world, fn, *args, timeout=300):
    """fn(rank, world, comm, stream, *args) -> result; returns the list of results."""
    from asystem_amem_b200 import Communicator, get_unique_id
    uid = get_unique_id()
    results = [None] * world
    errors = [None] * world

    def body(rank):
        try:
            torch.cuda.set_device(0)
            comm = Communicator(world, rank, uid)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                results[rank] = fn(rank, world, comm, stream, *args)
            stream.synchronize()
            err = comm.async_error()
            assert err == 0, f"device-side error {err}"
            comm.destroy()
        except BaseException as e:  # noqa: BLE001
            errors[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout)
    for r in range(world):
        assert not threads[r].is_alive(), f"rank {r} did not finish"
        assert errors[r] is None, f"rank {r}: {errors[r]}"
    return results
