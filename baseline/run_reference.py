"""Run the UNMODIFIED reference's raw-collective benchmark on its NCCL branch and report its times.

    python baseline/run_reference.py all_gather     [--json out.json]      # one GPU
    torchrun --nproc-per-node 8 baseline/run_reference.py reduce_scatter   # eight GPUs

What runs is ``baseline/_ref/benchmark_raw_collectives/{all_gather,reduce_scatter}.py`` of the
reference, byte for byte, started as ``__main__`` with

    --num-gpus-per-node N --machine b200 --library xccl --pccl-disable-cpp-backend

which is its NCCL build: ``pg = None; function = _all_gather`` / ``_reduce_scatter``
(``benchmark_raw_collectives/all_gather.py:67-69``, ``reduce_scatter.py:67-69``), ending in
``dist.all_gather_into_tensor`` / ``dist.reduce_scatter_tensor`` on the world group
(``pccl/all_gather.py:108-110``, ``pccl/reduce_scatter.py:175-180``) and timed by the
reference's own ``time_something`` (``benchmark_raw_collectives/utils.py:16-33``: 5 warm-up
calls, 20 timed calls between one pair of CUDA events, mean, rank 0).  Nothing of this
repository's library is imported in this process.

Two things are provided from outside, neither of which the timed branch executes:
``mpi4py`` is replaced by the import stand-in under ``baseline/stubs`` (the reference imports it
in every module), and ``SLURM_PROCID`` / ``SLURM_NTASKS`` are set from torchrun's ``RANK`` /
``WORLD_SIZE`` because the reference reads its rank from SLURM (``utils.py:7-8``).

The reference writes ``./data/<collective>/b200/gpus_<N>_slurm_<job>.csv`` relative to the
working directory; this runner changes into a scratch directory first, reads the CSV back and
prints one JSON line on rank 0:

    {"impl": "reference", "collective": "all_gather", "n_gpus": 8, "dtype": "bf16",
     "size_mode": "total_output", "rows": [{"size_mib": 1, "time_ms": ...}, ...]}
"""
from __future__ import annotations

import csv
import json
import os
import runpy
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
STUBS = HERE / "stubs"


def reference_available() -> str:
    """Empty string when the reference tree is present, else the reason it cannot run."""
    if not (REF / "benchmark_raw_collectives" / "all_gather.py").exists():
        return "baseline/_ref does not hold the reference tree (copy the reference repository there)"
    return ""


def main() -> int:
    argv = sys.argv[1:]
    if not argv or argv[0] not in ("all_gather", "reduce_scatter"):
        print("usage: run_reference.py {all_gather|reduce_scatter} [--json PATH] [--dtype bf16|fp32]", file=sys.stderr)
        return 2
    kind = argv[0]
    json_path = None
    dtype = "bf16" if kind == "all_gather" else "fp32"      # the reduce-scatter script is fp32 only
    i = 1
    while i < len(argv):
        if argv[i] == "--json":
            json_path, i = argv[i + 1], i + 2
        elif argv[i] == "--dtype" and kind == "all_gather":
            dtype, i = argv[i + 1], i + 2
        else:
            print(f"unknown argument {argv[i]}", file=sys.stderr)
            return 2
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    why = reference_available()
    if why:
        if rank == 0:
            print(json.dumps({"impl": "reference", "collective": kind, "unavailable": why}))
        return 0
    os.environ["SLURM_PROCID"] = str(rank)
    os.environ["SLURM_NTASKS"] = str(world)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if json_path is not None:
        json_path = str(Path(json_path).resolve())
    script = REF / "benchmark_raw_collectives" / f"{kind}.py"
    # the reference's packages first, the stand-in for mpi4py next; the reduce-scatter script
    # imports `utils` from its own directory
    sys.path[:0] = [str(script.parent), str(REF), str(STUBS)]
    scratch = tempfile.mkdtemp(prefix=f"pccl_ref_{kind}_r{rank}_")
    os.chdir(scratch)
    sys.argv = [str(script), "--num-gpus-per-node", str(world), "--machine", "b200", "--library", "xccl",
                "--pccl-disable-cpp-backend"]
    if kind == "all_gather":
        sys.argv += ["--dtype", dtype]
    runpy.run_path(str(script), run_name="__main__")
    if rank == 0:
        rows = []
        files = sorted(Path(scratch, "data", kind, "b200").glob("*.csv"))
        for f in files:
            with open(f, newline="") as fh:
                for rec in csv.DictReader(fh):
                    rows.append({"size_mib": float(rec["output_size"]), "time_ms": float(rec["time_xccl"])})
        out = {"impl": "reference", "collective": kind, "n_gpus": world, "dtype": dtype,
               "size_mode": "total_output" if kind == "all_gather" else "total_input",
               "timing": "reference's time_something: 5 warm-up + 20 timed calls, one CUDA-event pair, mean, rank 0",
               "rows": rows}
        line = json.dumps(out)
        print(line)
        if json_path is not None:
            Path(json_path).parent.mkdir(parents=True, exist_ok=True)
            Path(json_path).write_text(line + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
