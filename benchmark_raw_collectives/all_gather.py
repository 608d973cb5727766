"""All-gather bandwidth sweep and correctness check.

Command line of ``benchmark_raw_collectives/all_gather.py`` in the reference
(``--num-gpus-per-node --machine --library {pccl,mpi,xccl} --pccl-disable-cpp-backend
--test --pccl-recursive-alg --dtype``), plus ``--algorithm``, ``--sizes``, ``--size-mode``,
``--symmetric``, ``--nvls``, ``--json``, ``--write-tuning-table`` and ``--impl reference`` (which hands
over to ``baseline/run_reference.py``: the unmodified reference on its NCCL branch).  ``--library xccl`` (also spelled ``rccl`` / ``nccl``) is the
reference's NCCL path, ``dist.all_gather_into_tensor`` on the world group; ``mpi`` is not
available here (no MPI implementation) and is refused.

Two sweeps:
  ``--size-mode output``  the reference's (``benchmark_raw_collectives/all_gather.py:54-55,86-92``):
                          TOTAL OUTPUT 1..1024 MiB, per-rank input = output / world
  ``--size-mode input``   PER-RANK INPUT 1 MiB..1 GiB (default)
Times are device-timed, 5 warm-up + 20 timed calls, maximum over ranks; every row reports bus
bandwidth and its fraction of the 900 GB/s per-direction NVLink roofline.

    torchrun --nproc-per-node 8 benchmark_raw_collectives/all_gather.py \
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

from benchmark_raw_collectives.utils import (NVLINK_GBS_NOMINAL, CsvLog, allclose, bus_bandwidth_gbs, init,  # noqa: E402
                                             parse_sizes, sizes_pow2, time_something, update_tuning_table)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--num-gpus-per-node", type=int, required=True)
    ap.add_argument("--machine", type=str, required=True)
    ap.add_argument("--library", type=str, default="pccl", choices=["pccl", "mpi", "xccl", "rccl", "nccl"])
    ap.add_argument("--pccl-disable-cpp-backend", dest="use_pccl_cpp_backend", action="store_false")
    ap.add_argument("--test", action="store_true")
    ap.add_argument("--pccl-recursive-alg", action="store_true")
    ap.add_argument("--dtype", type=str, default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--algorithm", type=str, default=None,
                    help="direct|ring|recursive|pull|multimem|auto|all (overrides --pccl-recursive-alg)")
    ap.add_argument("--sizes", type=str, default=None, help="comma list, e.g. 1M,64M,1G")
    ap.add_argument("--size-mode", type=str, default="input", choices=["input", "output"])
    ap.add_argument("--symmetric", type=int, default=1, help="1: buffers in the symmetric heap (zero-copy)")
    ap.add_argument("--lanes", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", type=str, default=None, help="write all rows to this file (rank 0)")
    ap.add_argument("--nvls", type=int, default=None, help="1: bind an NVLS multicast mapping (multimem variant)")
    ap.add_argument("--write-tuning-table", type=str, default=None, metavar="PATH",
                    help="with --algorithm all: replace this group size's all-gather rows of the tuner's table")
    ap.add_argument("--impl", type=str, default="pccl", choices=["pccl", "reference"],
                    help="reference: run the unmodified reference benchmark (its --library xccl branch) instead")
    args = ap.parse_args()
    if args.impl == "reference":
        runner = str(Path(__file__).resolve().parent.parent / "baseline" / "run_reference.py")
        cmd = [sys.executable, runner, "all_gather", "--dtype", args.dtype] + (["--json", args.json] if args.json else [])
        os.execv(sys.executable, cmd)
    if args.library == "mpi":
        raise SystemExit("--library mpi: no MPI implementation is installed on this machine")

    rank, world = init()
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    es = 2 if dtype == torch.bfloat16 else 4
    baseline = args.library in ("xccl", "rccl", "nccl")
    if args.size_mode == "output":
        sizes = [s // world for s in parse_sizes(args.sizes, sizes_pow2(1 << 20, 1 << 30))]
    else:
        sizes = parse_sizes(args.sizes, sizes_pow2(1 << 20, 1 << 30))
    max_in = max(sizes)

    import pccl
    from pccl import schedule as sch

    comm = group = None
    if not baseline:
        from pccl import build_kernels

        build_kernels.build_rank0_first(dist.barrier)     # rank 0 compiles first, like the reference's callers
        heap = (world + 1) * max_in + (256 << 20) + (64 << 20) if args.symmetric else (512 << 20)
        comm = pccl.init(heap_bytes=heap, staging_bytes=256 << 20,
                         enable_nvls=None if args.nvls is None else bool(args.nvls))
        pgs = pccl.ProcessGroups(args.num_gpus_per_node, world // args.num_gpus_per_node)
        group = pgs.get_flat_group()
    if args.algorithm == "all":
        algos = [sch.DIRECT, sch.RING, sch.PULL] + ([sch.RECURSIVE] if sch.is_pow2(world) else [])
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
    log = CsvLog("all_gather", args.machine, world, cols, rank == 0)
    rows = []
    ok_all = True
    for n_bytes in sizes:
        n = n_bytes // es
        if not baseline and args.symmetric:
            out = comm.empty(world * n, dtype)
            inp = comm.empty(n, dtype)
        else:
            out = torch.empty(world * n, dtype=dtype, device=dev)
            inp = torch.empty(n, dtype=dtype, device=dev)
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        inp.copy_(torch.randn(n, generator=gen, device=dev, dtype=torch.float32).to(dtype))
        for algo in algos:
            if baseline:
                fn = lambda: pccl._all_gather(out, inp, None)  # noqa: E731
            else:
                fn = lambda a=algo: pccl._all_gather(out, inp, group, use_rd=(a == sch.RECURSIVE),  # noqa: E731
                                                     use_pccl_cpp_backend=args.use_pccl_cpp_backend, algorithm=a,
                                                     lanes=args.lanes)
            ms = time_something(fn, warmup_iters=args.warmup, timed_iters=args.iters)
            if comm is not None:
                comm.check()
            if args.test:
                gold = torch.empty(world * n, dtype=dtype, device=dev)
                pccl._all_gather(gold, inp, None)
                out.zero_()
                fn()
                torch.cuda.synchronize()
                good = torch.equal(out, gold) if not baseline else allclose(out, gold)
                flag = torch.tensor([1 if good else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                ok_all = ok_all and bool(flag.item())
                del gold
            bw = bus_bandwidth_gbs(n_bytes, world, ms)
            row = {"gpu_count": world, "slurm_job_id": os.environ.get("SLURM_JOB_ID", "local"),
                   "output_size": world * n_bytes / (1 << 20), "unit": "MiB", "library": label, "algorithm": algo,
                   "per_rank_bytes": n_bytes, "time_ms": round(ms, 5), "busbw_gbs": round(bw, 2),
                   "frac_of_900": round(bw / NVLINK_GBS_NOMINAL, 4)}
            rows.append(row)
            log.row(row)
            if rank == 0:
                print(f"all_gather P={world} per-rank {n_bytes / (1 << 20):9.3f} MiB {label:9s} {algo:9s} "
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
            pt = pts.setdefault(r["per_rank_bytes"], {"collective": "all_gather", "P": world,
                                                      "per_rank_bytes": r["per_rank_bytes"], "variants": {}})
            pt["variants"][r["algorithm"]] = {"ms": r["time_ms"]}
        update_tuning_table(Path(args.write_tuning_table), "all_gather", world, list(pts.values()))
    dist.barrier()
    if comm is not None:
        pccl.shutdown()
    dist.destroy_process_group()
    if args.test and not ok_all:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
