"""Pure-Python statement of the collective schedules.

This module is the host-side twin of ``pccl/csrc/schedule.h``: the CPU (gloo) backend runs
these schedules over point-to-point messages, and the unit tests cross-check the two
implementations step by step.  It deliberately shares no code with the header.

Reference parity: recursive doubling is the schedule of ``pccl/all_gather.py:52-90``,
recursive halving that of ``pccl/reduce_scatter.py:62-97`` and the ring reduce-scatter
that of ``pccl/reduce_scatter.py:138-160`` in the reference.  The reference has no ring
all-gather of its own (it calls the vendor MPI) and no direct variant.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

DIRECT = "direct"
RING = "ring"
RECURSIVE = "recursive"
PULL = "pull"
MULTIMEM = "multimem"
AUTO = "auto"
# all-gather only: peer-to-local copies by the GPU's copy engines, no kernel and no handshake; the
# caller guarantees that the peers' inputs do not change while the call is in flight
COPY_ENGINE = "copy_engine"

# small messages on the world group: the direct schedule into a double-buffered landing area of the
# communicator without the entry handshake (one flag trip instead of three)
EAGER = "eager"

ALGO_IDS = {DIRECT: 0, RING: 1, RECURSIVE: 2, PULL: 3, MULTIMEM: 4, EAGER: 5}
ALGO_NAMES = {v: k for k, v in ALGO_IDS.items()}
MAX_RANKS = 8


@dataclass(frozen=True)
class Step:
    dst: int
    src: int
    send_first: int
    recv_first: int
    nblocks: int


def is_pow2(p: int) -> bool:
    return p > 0 and (p & (p - 1)) == 0


def check_algo(algo: str, world: int) -> None:
    """Recursive variants need a power-of-two group; the others accept any size."""
    if algo not in ALGO_IDS:
        raise ValueError(f"unknown algorithm {algo!r}; expected one of {sorted(ALGO_IDS)}")
    if algo == RECURSIVE and not is_pow2(world):
        raise ValueError(
            f"the recursive doubling/halving algorithms need a power-of-two group size, got {world}"
        )


def num_steps(algo: str, world: int) -> int:
    if world <= 1:
        return 0
    if algo == RECURSIVE:
        return world.bit_length() - 1
    return world - 1


def ag_step(algo: str, world: int, rank: int, t: int) -> Step:
    if algo == RING:
        return Step((rank + 1) % world, (rank - 1) % world, (rank - t) % world, (rank - t - 1) % world, 1)
    if algo == RECURSIVE:
        seg = 1 << t
        partner = rank ^ seg
        mine = rank - rank % seg
        theirs = partner - partner % seg
        return Step(partner, partner, mine, theirs, seg)
    src = (rank - 1 - t) % world
    return Step((rank + 1 + t) % world, src, rank, src, 1)


def rs_step(algo: str, world: int, rank: int, t: int) -> Step:
    if algo == RING:
        return Step((rank + 1) % world, (rank - 1) % world, (rank - t - 1) % world, (rank - t - 2) % world, 1)
    if algo == RECURSIVE:
        group = world >> t
        half = group // 2
        base = rank - rank % group
        if rank - base < half:
            return Step(rank + half, rank + half, base + half, base, half)
        return Step(rank - half, rank - half, base, base + half, half)
    dst = (rank + 1 + t) % world
    return Step(dst, (rank - 1 - t) % world, dst, rank, 1)


def rs_stage_offset(algo: str, world: int, t: int) -> int:
    if algo != RECURSIVE:
        return t
    return sum(world >> (j + 1) for j in range(t))


def rs_dep_steps(algo: str, world: int, t: int) -> List[int]:
    """Earlier steps whose received partial sums are folded into step ``t``'s payload
    (``t == num_steps`` names the final result)."""
    n = num_steps(algo, world)
    if algo == RING:
        return [] if t == 0 else [t - 1]
    if algo == RECURSIVE:
        return list(range(t))
    return list(range(n)) if t == n else []


def grid_coords(world_rank: int, intra: int, inter: int):
    """(grid, outer, inner) of a world rank; inner ranks are consecutive."""
    return world_rank // (intra * inter), (world_rank // intra) % inter, world_rank % intra
