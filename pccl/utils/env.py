"""Rank discovery and process-group start-up.

The reference reads ``SLURM_PROCID`` / ``SLURM_NTASKS`` and calls
``init_process_group("nccl", env://)`` (``benchmark_raw_collectives/utils.py:6-13``); its
launch scripts export ``MASTER_ADDR`` / ``MASTER_PORT`` / ``WORLD_SIZE``
(``scripts/perlmutter/run_raw_collectives_benchmark.sh:17-30``).  Here torchrun's
``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK`` come first, the SLURM names are the fallback,
and a lone process becomes a world of one.
"""
from __future__ import annotations

import datetime
import os
import socket
from typing import Tuple

import torch
import torch.distributed as dist


def discover() -> Tuple[int, int, int]:
    """(rank, world, local_rank) from the environment."""
    env = os.environ
    rank = int(env.get("RANK", env.get("SLURM_PROCID", "0")))
    world = int(env.get("WORLD_SIZE", env.get("SLURM_NTASKS", "1")))
    local = int(env.get("LOCAL_RANK", env.get("SLURM_LOCALID", str(rank))))
    return rank, world, local


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def init_distributed(backend: str = None, timeout_s: float = 600.0) -> Tuple[int, int, int]:
    """Initialise torch.distributed (NCCL on GPUs, gloo otherwise) and bind this process to
    its GPU.  Returns (rank, world, local_rank)."""
    rank, world, local = discover()
    if torch.cuda.is_available():
        ndev = torch.cuda.device_count()
        torch.cuda.set_device(local % ndev)
    if dist.is_initialized():
        return rank, world, local
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        if world != 1:
            raise RuntimeError("MASTER_PORT must be set when WORLD_SIZE > 1")
        os.environ["MASTER_PORT"] = str(_free_port())
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world, local
