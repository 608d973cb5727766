"""Run a function on `world` CPU processes connected by gloo (127.0.0.1 rendezvous)."""
import datetime
import os
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, port, fn, args, backend, errq):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["LOCAL_RANK"] = str(rank)
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
        fn(rank, world, *args)
        errq.put((rank, None))
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def run_ranks(fn, world, port, args=(), backend="gloo", timeout=120):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, backend, errq)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _queue

    results = []
    timed_out = False
    try:
        for _ in range(world):
            try:
                # once one rank has failed, its peers are probably stuck in a collective: do not wait long
                failed = any(tb is not None for _r, tb in results)
                results.append(errq.get(timeout=15 if failed else timeout))
            except _queue.Empty:
                timed_out = True
                break
    finally:
        for p in procs:
            p.join(timeout=1 if timed_out else 10)
            if p.is_alive():
                p.kill()   # exact child we started
    failures = [f"rank {r}:\n{tb}" for r, tb in results if tb is not None]
    assert not failures, "\n".join(failures)
    assert not timed_out, f"only {len(results)} of {world} ranks finished within the time limit"
    assert len(results) == world
