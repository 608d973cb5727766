"""Reduce-scatter (SUM) bandwidth sweep and correctness check.

Command line of ``benchmark_raw_collectives/reduce_scatter.py`` in the reference, plus
``--algorithm``, ``--sizes``, ``--size-mode``, ``--dtype``, ``--out-dtype``, ``--symmetric``, ``--nvls``,
``--json``, ``--write-tuning-table`` and ``--impl reference`` (hands over to
``baseline/run_reference.py``: the unmodified reference on its NCCL branch).  Unlike
the reference (which always passes ``use_rh=True`` whatever the flag says, line 95), the
algorithm flag is respected.  ``--library xccl|rccl|nccl`` is ``dist.reduce_scatter_tensor``
on the world group.

Sizes are the PER-RANK INPUT buffer (default bf16, 8 MiB..8 GiB); every rank's result is
input / world.  The reference's own sweep is ``--dtype fp32 --sizes 1M,2M,...,1G`` (it calls the
same quantity the total input, ``benchmark_raw_collectives/reduce_scatter.py:86-90``).
bf16 inputs are summed with fp32 accumulation.  Times are device-timed, maximum over ranks;
bus bandwidth = (P-1)/P * input bytes / time.

    torchrun --nproc-per-node 8 benchmark_raw_collectives/reduce_scatter.py \
        --num-gpus-per-node 8 --machine b200 --library pccl --algorithm all --test
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from benchmark_raw_collectives.utils import (NVLINK_GBS_NOMINAL, CsvLog, init, parse_sizes, sizes_pow2,  # noqa: E402
                                             time_something, update_tuning_table)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--num-gpus-per-node", type=int, required=True)
    ap.add_argument("--machine", type=str, required=True)
    ap.add_argument("--library", type=str, default="pccl", choices=["pccl", "mpi", "xccl", "rccl", "nccl"])
    ap.add_argument("--pccl-disable-cpp-backend", dest="use_pccl_cpp_backend", action="store_false")
    ap.add_argument("--test", action="store_true")
    ap.add_argument("--pccl-recursive-alg", action="store_true")
    ap.add_argument("--dtype", type=str, default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--out-dtype", type=str, default=None, choices=[None, "bf16", "fp32"])
    ap.add_argument("--algorithm", type=str, default=None)
    ap.add_argument("--sizes", type=str, default=None)
    ap.add_argument("--symmetric", type=int, default=1)
    ap.add_argument("--lanes", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", type=str, default=None)
    ap.add_argument("--size-mode", type=str, default="input", choices=["input", "output"],
                    help="input: sizes are each rank's INPUT buffer (what the reference calls the total input); "
                         "output: sizes are the per-rank result, the input is world times larger")
    ap.add_argument("--nvls", type=int, default=None, help="1: bind an NVLS multicast mapping (multimem variant)")
    ap.add_argument("--write-tuning-table", type=str, default=None, metavar="PATH",
                    help="with --algorithm all: replace this group size's reduce-scatter rows of the tuner's table")
    ap.add_argument("--impl", type=str, default="pccl", choices=["pccl", "reference"],
                    help="reference: run the unmodified reference benchmark (its NCCL branch; fp32, total input 1..1024 MiB)")
    args = ap.parse_args()
    if args.impl == "reference":
        runner = str(Path(__file__).resolve().parent.parent / "baseline" / "run_reference.py")
        os.execv(sys.executable, [sys.executable, runner, "reduce_scatter"] + (["--json", args.json] if args.json else []))
    if args.library == "mpi":
        raise SystemExit("--library mpi: no MPI implementation is installed on this machine")

    rank, world = init()
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    out_dtype = dtype if args.out_dtype is None else (torch.bfloat16 if args.out_dtype == "bf16" else torch.float32)
    es = 2 if dtype == torch.bfloat16 else 4
    baseline = args.library in ("xccl", "rccl", "nccl")
    if baseline:
        out_dtype = dtype
    sizes = parse_sizes(args.sizes, sizes_pow2(8 << 20, 8 << 30))
    if args.size_mode == "output":
        sizes = [s * world for s in sizes]
    max_in = max(sizes)

    import pccl
    from pccl import schedule as sch

    comm = group = None
    if not baseline:
        from pccl import build_kernels

        build_kernels.build_rank0_first(dist.barrier)
        staging = max(256 << 20, max_in)             # push variants stage (P-1)/P of the input
        heap = (max_in + (64 << 20) if args.symmetric else (64 << 20)) + staging + (64 << 20)
        comm = pccl.init(heap_bytes=heap, staging_bytes=staging, enable_nvls=None if args.nvls is None else bool(args.nvls))
        pgs = pccl.ProcessGroups(args.num_gpus_per_node, world // args.num_gpus_per_node)
        group = pgs.get_flat_group()
    if args.algorithm == "all":
        algos = [sch.DIRECT, sch.RING] + ([sch.RECURSIVE] if sch.is_pow2(world) else [])
        if args.symmetric:
            algos.append(sch.PULL)
            if comm is not None and comm.nvls:
                algos.append(sch.MULTIMEM)
    elif args.algorithm:
        algos = [args.algorithm]
    else:
        algos = [sch.RECURSIVE if args.pccl_recursive_alg else sch.RING]
    if baseline:
        algos = ["nccl"]

    label = args.library + ("" if baseline else ("_cpp" if args.use_pccl_cpp_backend else "_py"))
    cols = ["gpu_count", "slurm_job_id", "output_size", "unit", "library", "algorithm", "per_rank_bytes", "time_ms",
            "busbw_gbs", "frac_of_900"]
    log = CsvLog("reduce_scatter", args.machine, world, cols, rank == 0)
    rows = []
    ok_all = True
    for in_bytes in sizes:
        n = in_bytes // es // world              # elements of the result
        if n == 0:
            continue
        if not baseline and args.symmetric:
            inp = comm.empty(world * n, dtype)
        else:
            inp = torch.empty(world * n, dtype=dtype, device=dev)
        out = torch.empty(n, dtype=out_dtype, device=dev)
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        chunk = 1 << 26
        for s in range(0, world * n, chunk):       # N(0,1) without a full-size fp32 temporary
            e = min(world * n, s + chunk)
            inp[s:e].copy_(torch.randn(e - s, generator=gen, device=dev, dtype=torch.float32).to(dtype))
        for algo in algos:
            if baseline:
                fn = lambda: pccl._reduce_scatter(out, inp, None)  # noqa: E731
            else:
                fn = lambda a=algo: pccl._reduce_scatter(out, inp, group, use_rh=(a == sch.RECURSIVE),  # noqa: E731
                                                         use_pccl_cpp_backend=args.use_pccl_cpp_backend, algorithm=a,
                                                         lanes=args.lanes)
            ms = time_something(fn, warmup_iters=args.warmup, timed_iters=args.iters)
            if comm is not None:
                comm.check()
            if args.test:
                gold = torch.empty(n, dtype=dtype, device=dev)
                pccl._reduce_scatter(gold, inp, None)
                fn()
                torch.cuda.synchronize()
                # NCCL rounds bf16 partial sums; compare in fp32 with a tolerance that covers it
                rtol, atol = (1e-5, 1e-5) if dtype == torch.float32 else (4e-2, 4e-2)
                close = torch.isclose(out.float(), gold.float(), rtol=rtol, atol=atol)
                good = float((~close).sum()) <= 0.02 * n
                flag = torch.tensor([1 if good else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                ok_all = ok_all and bool(flag.item())
                del gold
            bw = (world - 1) / world * in_bytes / (ms * 1e-3) / 1e9 if world > 1 else 0.0
            row = {"gpu_count": world, "slurm_job_id": os.environ.get("SLURM_JOB_ID", "local"),
                   "output_size": in_bytes / (1 << 20), "unit": "MiB", "library": label, "algorithm": algo,
                   "per_rank_bytes": in_bytes, "time_ms": round(ms, 5), "busbw_gbs": round(bw, 2),
                   "frac_of_900": round(bw / NVLINK_GBS_NOMINAL, 4)}
            rows.append(row)
            log.row(row)
            if rank == 0:
                print(f"reduce_scatter P={world} per-rank input {in_bytes / (1 << 20):9.3f} MiB {label:9s} {algo:9s} "
                      f"{ms * 1e3:10.1f} us  busbw {bw:7.1f} GB/s  ({100 * bw / NVLINK_GBS_NOMINAL:5.1f}% of 900)", flush=True)
        del out, inp
    if args.test and rank == 0:
        print("All tests passed! PCCL outputs match NCCL outputs!" if ok_all else "TEST FAILED: outputs differ from NCCL")
    if args.json and rank == 0:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))
    if args.write_tuning_table and rank == 0 and not baseline and len(algos) > 1:
        pts = {}
        for r in rows:
            pt = pts.setdefault(r["per_rank_bytes"], {"collective": "reduce_scatter", "P": world,
                                                      "per_rank_bytes": r["per_rank_bytes"], "variants": {}})
            pt["variants"][r["algorithm"]] = {"ms": r["time_ms"]}
        update_tuning_table(Path(args.write_tuning_table), "reduce_scatter", world, list(pts.values()))
    dist.barrier()
    if comm is not None:
        pccl.shutdown()
    dist.destroy_process_group()
    if args.test and not ok_all:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
