"""Shared pieces of the raw-collective benchmarks.

Keeps the helper names of ``benchmark_raw_collectives/utils.py`` in the reference
(``init``, ``time_something``, ``allclose``).  ``time_something`` is device-timed like the
reference's (one CUDA-event pair around the timed calls after warm-up) but returns the
MAXIMUM over ranks instead of rank 0's value, and the drivers turn times into bus
bandwidth and a fraction of the NVLink roofline, which the reference never computes.
"""
from __future__ import annotations

import csv
import os
import sys
from pathlib import Path
from typing import Dict, List, Optional

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from pccl.utils.env import init_distributed  # noqa: E402
from pccl.utils.timing import time_something  # noqa: E402,F401

NVLINK_GBS_NOMINAL = 900.0    # per direction per GPU
NVLINK_GBS_MEASURED = 770.0   # peer copy measured on this pool


def init():
    """Start torch.distributed from torchrun or SLURM variables; returns (rank, world)."""
    rank, world, _local = init_distributed()
    return rank, world


def allclose(x: torch.Tensor, y: torch.Tensor, pct: float = 2.0) -> bool:
    """``isclose(rtol=1e-5)`` with at most ``pct`` percent of elements allowed to differ: the
    tolerance rule of the reference's ``--test`` (``benchmark_raw_collectives/utils.py:35-42``)."""
    close = torch.isclose(x.float(), y.float(), rtol=1e-5)
    bad = 100.0 * float((~close).sum()) / max(1, x.numel())
    if bad > pct:
        print(f"mismatch: {bad:.3f}% of elements differ")
        return False
    return True


def bus_bandwidth_gbs(per_rank_bytes: int, world: int, ms: float) -> float:
    """busbw = (P-1)/P * total bytes / time, with total = P * per-rank bytes."""
    if ms <= 0 or world <= 1:
        return 0.0
    return (world - 1) * per_rank_bytes / (ms * 1e-3) / 1e9


def sizes_pow2(lo: int, hi: int) -> List[int]:
    out, s = [], lo
    while s <= hi:
        out.append(s)
        s *= 2
    return out


def parse_sizes(text: Optional[str], default: List[int]) -> List[int]:
    if not text:
        return default
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    out = []
    for tok in text.split(","):
        tok = tok.strip().upper()
        m = 1
        if tok and tok[-1] in mult:
            m, tok = mult[tok[-1]], tok[:-1]
        out.append(int(float(tok) * m))
    return out


def job_id() -> str:
    return os.environ.get("SLURM_JOB_ID", os.environ.get("TORCHELASTIC_RUN_ID", "local"))


class CsvLog:
    """Rank 0 appends rows to ./data/<collective>/<machine>/gpus_<N>_slurm_<job>.csv."""

    def __init__(self, collective: str, machine: str, world: int, columns: List[str], enabled: bool):
        self.enabled = enabled
        self.columns = columns
        if not enabled:
            return
        folder = Path("data") / collective / machine
        folder.mkdir(parents=True, exist_ok=True)
        self.path = folder / f"gpus_{world}_slurm_{job_id()}.csv"
        new = not self.path.exists()
        self.fh = open(self.path, "a", newline="")
        self.w = csv.writer(self.fh)
        if new:
            self.w.writerow(columns)

    def row(self, values: Dict) -> None:
        if self.enabled:
            self.w.writerow([values.get(c, "") for c in self.columns])
            self.fh.flush()


def tuning_rows(points: List[Dict]) -> List[List]:
    """Turn measured points of one collective and group size into rows of the tuner's table.

    ``points``: dictionaries with ``per_rank_bytes``, the tuner's key (all-gather: bytes each rank
    contributes; reduce-scatter: bytes of the per-rank INPUT BUFFER, converted here to the result
    block the tuner is asked about) and ``variants`` = {name: {"ms": ...}}.  For every size the
    preference list is every measured variant, fastest first (the tuner takes the first one the
    tensors' placement allows, so a private input or a missing multicast mapping falls to the next
    best instead of to a fixed default), with ``direct``, which every placement can run, at the
    latest as the last entry.  Neighbouring sizes whose first three preferences agree share a row; a
    row covers sizes up to and including its ``max_bytes``, the last one everything above."""
    pts = sorted(points, key=lambda p: p["per_rank_bytes"])
    rows: List[List] = []
    for p in pts:
        prefs = sorted(p["variants"], key=lambda a: p["variants"][a]["ms"])
        if "direct" not in prefs:
            prefs.append("direct")
        key_bytes = p["per_rank_bytes"]
        is_rs = p["collective"] == "reduce_scatter"
        if is_rs:
            key_bytes //= p["P"]
        # small all-gathers: at most 32 lanes; reduce-scatters take 64 throughout (the tuner still caps by size)
        lanes = 32 if key_bytes <= (4 << 20) and not is_rs else 64
        if rows and rows[-1][1][:3] == prefs[:3] and rows[-1][2] == lanes:
            rows[-1][0] = key_bytes
        else:
            rows.append([key_bytes, prefs, lanes])
    if rows:
        rows[-1][0] = None
    return rows


def update_tuning_table(path: Path, collective: str, world: int, points: List[Dict]) -> None:
    """Replace the rows of (collective, world) in the JSON table at ``path`` with the winners of
    ``points``; everything else in the file is kept."""
    import json

    table: Dict = {}
    if path.exists():
        try:
            table = json.loads(path.read_text())
        except ValueError:
            table = {}
    table.setdefault(collective, {})[str(world)] = tuning_rows(points)
    table["_comment"] = ("size x group -> preferred variants (first feasible wins) and lanes; written by "
                         "benchmark_raw_collectives/sweep.py --write-tuning-table from device-timed, max-over-ranks times")
    path.write_text(json.dumps(table, indent=1) + "\n")
