"""Pick the algorithm variant and the number of lanes for one collective call.

``algorithm="auto"`` consults a table keyed by collective, group size and message size
that is produced from measured bus bandwidth (``benchmark_raw_collectives/sweep.py`` and the
two per-collective drivers write it with ``--write-tuning-table``).  The reference has no such
choice: its caller passes
``use_rd`` / ``use_rh`` by hand (``pccl/all_gather.py:98-105``) and its README only says
that the recursive variants are "typically faster at scale".

Environment overrides: ``PCCL_ALGO`` (direct|ring|recursive|pull|multimem) and
``PCCL_LANES`` (integer) win over the table.
"""
from __future__ import annotations

import json
import os
from functools import lru_cache
from pathlib import Path
from typing import Dict, List, Optional, Tuple

from . import schedule as sch

TABLE_PATH = Path(__file__).resolve().parent / "tuning_table.json"

# Fallback when the table has no row: bytes each lane should at least move, lane ceiling.
MIN_BYTES_PER_LANE = 64 << 10
PIPELINE_BYTES_PER_LANE = 256 << 10   # per-lane share that fills the bulk-copy pipeline (the kernels switch to it at 192 KiB)
DEFAULT_MAX_LANES = 148


@lru_cache(maxsize=1)
def _table() -> Dict:
    if TABLE_PATH.exists():
        try:
            return json.loads(TABLE_PATH.read_text())
        except (OSError, ValueError):
            return {}
    return {}


def reload_table() -> None:
    _table.cache_clear()


def default_lanes(nbytes: int, max_lanes: int = DEFAULT_MAX_LANES) -> int:
    lanes = max(1, min(max_lanes, nbytes // MIN_BYTES_PER_LANE))
    return int(lanes)


def lookup(collective: str, world: int, nbytes: int) -> Optional[Tuple[List[str], int]]:
    """Row of the table for this size: (variants in order of preference, lanes)."""
    rows: List = _table().get(collective, {}).get(str(world), [])
    for max_bytes, algos, lanes in rows:
        if max_bytes is None or nbytes <= max_bytes:
            return ([algos] if isinstance(algos, str) else list(algos)), int(lanes)
    return None


def _feasible(collective: str, algo: str, world: int, nbytes: int, symmetric_in: bool, symmetric_out: bool,
              has_multimem: bool, eager_capacity: int = 0) -> bool:
    """Variants that read or multicast peer memory need the right tensors in the heap."""
    if algo == sch.EAGER:
        # eager_capacity is 0 unless the call is on the world group of a communicator with an eager area
        need = world * nbytes if collective == "all_gather" else (world - 1) * nbytes
        return collective in ("all_gather", "reduce_scatter") and 0 < need <= eager_capacity
    if algo == sch.MULTIMEM:
        if not has_multimem or nbytes % 16 != 0:
            return False
        if collective == "all_gather" and not symmetric_out:
            return False
        if collective in ("reduce_scatter", "all_reduce") and not symmetric_in:
            return False
    if collective == "reduce_scatter" and algo == sch.PULL and not symmetric_in:
        return False
    if algo == sch.RECURSIVE and not sch.is_pow2(world):
        return False
    return True


def choose(collective: str, world: int, nbytes: int, *, requested: str = sch.AUTO, symmetric_in: bool = False,
           symmetric_out: bool = False, has_multimem: bool = False, lanes: Optional[int] = None,
           max_lanes: int = DEFAULT_MAX_LANES, eager_capacity: int = 0) -> Tuple[str, int]:
    """Return ``(algorithm, nlanes)``.  ``nbytes`` is the per-rank block size."""
    env_algo = os.environ.get("PCCL_ALGO")
    env_lanes = os.environ.get("PCCL_LANES")
    algo = requested
    if algo == sch.AUTO and env_algo:
        algo = env_algo
    picked_lanes = None
    if algo == sch.AUTO:
        hit = lookup(collective, world, nbytes)
        candidates, picked_lanes = hit if hit is not None else ([sch.DIRECT], None)
        algo = sch.DIRECT
        for cand in candidates:
            if _feasible(collective, cand, world, nbytes, symmetric_in, symmetric_out, has_multimem, eager_capacity):
                algo = cand
                break
    elif not _feasible(collective, algo, world, nbytes, symmetric_in, symmetric_out, has_multimem, eager_capacity):
        if algo == sch.RECURSIVE and requested == sch.RECURSIVE:
            sch.check_algo(algo, world)   # raises: the caller asked for it explicitly
        algo = sch.DIRECT
    if lanes is None:
        # A lane of a reduce-scatter reads its share of the block from every peer, and below the bulk-copy
        # threshold it does so in dependent rounds of a few vectors per thread: the share shrinks with the
        # number of peers (measured at P = 4: 256 KiB blocks, 16 lanes 31 us, 4 lanes 42 us).
        peer_reads = collective == "reduce_scatter" and algo != sch.MULTIMEM      # the switch variant reads once
        scaled = nbytes * max(1, world - 1) if peer_reads else nbytes
        lanes = int(env_lanes) if env_lanes else min(picked_lanes or 64, default_lanes(scaled, max_lanes))
        if collective == "reduce_scatter" and not env_lanes and lanes > 0 and algo != sch.MULTIMEM:
            # Shares between 64 KiB and 256 KiB are the slow zone of the peer-memory variants: below 192 KiB a
            # lane runs thread loops in dependent rounds, and at 192 KiB the bulk-copy pipeline is too short to
            # fill (measured at P = 4: 8 MiB blocks, 64 lanes 104 us, 32 lanes 65 us; 12 MiB blocks at exactly
            # 192 KiB per lane 132 us against 106 us for 16 MiB blocks at 256 KiB).  Take fewer lanes of 256 KiB
            # each, but never fewer than 32: below that the lanes themselves bound the bandwidth.
            share = nbytes // lanes
            fewer = nbytes // PIPELINE_BYTES_PER_LANE
            if MIN_BYTES_PER_LANE < share < PIPELINE_BYTES_PER_LANE and fewer >= 32:
                lanes = fewer
    return algo, max(1, min(int(lanes), max_lanes))
