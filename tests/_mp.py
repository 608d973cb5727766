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
    results = []
    try:
        for _ in range(world):
            results.append(errq.get(timeout=timeout))
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()   # exact child we started
    failures = [f"rank {r}:\n{tb}" for r, tb in results if tb is not None]
    assert not failures, "\n".join(failures)
    assert len(results) == world
