"""Both bandwidth sweeps in one launch: every variant of this library and NCCL, side by side.

    torchrun --nproc-per-node 8 benchmark_raw_collectives/sweep.py --test \
        --json out/sweep_p8.json --md out/sweep_p8.md --write-tuning-table pccl/tuning_table.json

Four sweeps (``--sweeps`` picks a subset):

  ``ag``      all-gather, bf16, PER-RANK INPUT 1 MiB .. 1 GiB in powers of two
  ``rs``      reduce-scatter, bf16 in / bf16 out with fp32 accumulation, PER-RANK INPUT BUFFER
              8 MiB .. 8 GiB in powers of two
  ``ag-ref``  the reference's own all-gather sweep: TOTAL OUTPUT 1 .. 1024 MiB, bf16
              (``benchmark_raw_collectives/all_gather.py:54-55,86-92`` of the reference)
  ``rs-ref``  the reference's own reduce-scatter sweep: TOTAL INPUT 1 .. 1024 MiB, fp32
              (``benchmark_raw_collectives/reduce_scatter.py:54,86-90`` of the reference)

Every point is timed like the reference times (``benchmark_raw_collectives/utils.py:16-33``:
5 warm-up calls, then 20 calls between one pair of CUDA events) but reported as the maximum
over the ranks.  The NCCL column is ``dist.all_gather_into_tensor`` /
``dist.reduce_scatter_tensor`` on the world group, the two calls the reference's
``--library xccl`` branch ends in; ``baseline/run_reference.py`` times the unmodified
reference itself for the ``*-ref`` shapes.

The communicator is created with NVLS when the machine offers it (``--nvls 1``, the default
here), so the multimem variants are measured in the same run; the plain variants do not use
the multicast mapping, and the report gives the best variant with and without multimem.
``--write-tuning-table`` replaces this group size's rows of the tuner's table with the
measured winners.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Dict, List

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from benchmark_raw_collectives.utils import (NVLINK_GBS_MEASURED, NVLINK_GBS_NOMINAL, init, parse_sizes,  # noqa: E402
                                             sizes_pow2, time_something, update_tuning_table)


def _fill_randn(t: torch.Tensor, seed: int) -> None:
    """N(0,1) values without a full-size fp32 temporary."""
    gen = torch.Generator(device=t.device).manual_seed(seed)
    chunk = 1 << 26
    for s in range(0, t.numel(), chunk):
        e = min(t.numel(), s + chunk)
        t[s:e].copy_(torch.randn(e - s, generator=gen, device=t.device, dtype=torch.float32).to(t.dtype))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweeps", default="ag,rs,ag-ref,rs-ref")
    ap.add_argument("--ag-sizes", default=None, help="per-rank input sizes, e.g. 1M,64M,1G (default 1M..1G)")
    ap.add_argument("--rs-sizes", default=None, help="per-rank input buffer sizes (default 8M..8G)")
    ap.add_argument("--algorithms", default="all", help="comma list or 'all'")
    ap.add_argument("--nvls", type=int, default=1)
    ap.add_argument("--lanes", default=None,
                    help="lanes (CTAs) per call; a comma list times every variant at every count (rows named variant@lanes)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--test", action="store_true", help="check every variant against NCCL at every size")
    ap.add_argument("--json", default=None)
    ap.add_argument("--md", default=None)
    ap.add_argument("--write-tuning-table", default=None, metavar="PATH")
    args = ap.parse_args()

    rank, world = init()
    dev = torch.device("cuda", torch.cuda.current_device())
    import pccl
    from pccl import build_kernels
    from pccl import schedule as sch

    sweeps = [s for s in args.sweeps.split(",") if s]
    ag_sizes = parse_sizes(args.ag_sizes, sizes_pow2(1 << 20, 1 << 30))
    rs_sizes = parse_sizes(args.rs_sizes, sizes_pow2(8 << 20, 8 << 30))
    ref_sizes = sizes_pow2(1 << 20, 1 << 30)
    plan = []          # (sweep, collective, dtype, per-rank input bytes of the call)
    for s in sweeps:
        if s == "ag":
            plan += [("ag", "all_gather", torch.bfloat16, b) for b in ag_sizes]
        elif s == "rs":
            plan += [("rs", "reduce_scatter", torch.bfloat16, b) for b in rs_sizes]
        elif s == "ag-ref":
            plan += [("ag-ref", "all_gather", torch.bfloat16, b // world) for b in ref_sizes]
        elif s == "rs-ref":
            plan += [("rs-ref", "reduce_scatter", torch.float32, b) for b in ref_sizes]
        else:
            raise SystemExit(f"unknown sweep {s!r}")
    max_ag = max([b for _s, c, _d, b in plan if c == "all_gather"] or [0])
    max_rs = max([b for _s, c, _d, b in plan if c == "reduce_scatter"] or [0])
    # symmetric buffers: all-gather output + input, reduce-scatter input; push variants of the
    # reduce-scatter stage (P-1)/P of the input in the receiver's staging area
    staging = max(256 << 20, max_rs)
    heap = max((world + 1) * max_ag, max_rs) + staging + (256 << 20)
    build_kernels.build_rank0_first(dist.barrier)
    comm = pccl.init(heap_bytes=heap, staging_bytes=staging, enable_nvls=bool(args.nvls))
    group = comm.world_group

    def variants(collective: str) -> List[str]:
        if args.algorithms != "all":
            return [a for a in args.algorithms.split(",") if a]
        v = [sch.DIRECT, sch.RING, sch.PULL] + ([sch.RECURSIVE] if sch.is_pow2(world) else [])
        if comm.nvls:
            v.append(sch.MULTIMEM)
        return v

    lane_counts = [int(x) for x in str(args.lanes).split(",") if x] if args.lanes else [None]
    if len(lane_counts) > 1 and args.write_tuning_table:
        raise SystemExit("--write-tuning-table needs one lane count (or none), not a list")
    rows: List[Dict] = []
    ok_all = True
    for sweep, collective, dtype, nbytes in plan:
        es = 2 if dtype == torch.bfloat16 else 4
        if collective == "all_gather":
            n = nbytes // es
            inp = comm.empty(n, dtype)
            out = comm.empty(world * n, dtype)
            _fill_randn(inp, 1234 + rank)
            gold = torch.empty(world * n, dtype=dtype, device=dev) if args.test else None

            def nccl():
                dist.all_gather_into_tensor(gold if gold is not None else out, inp)

            def ours(a, lanes=None):
                return lambda: pccl._all_gather(out, inp, group, use_pccl_cpp_backend=True, algorithm=a, lanes=lanes)

            wire = nbytes                                   # bytes every rank contributes
        else:
            n = nbytes // es // world                        # elements of the result
            if n == 0:
                continue
            inp = comm.empty(world * n, dtype)
            out = torch.empty(n, dtype=dtype, device=dev)
            _fill_randn(inp, 1234 + rank)
            gold = torch.empty(n, dtype=dtype, device=dev)

            def nccl():
                dist.reduce_scatter_tensor(gold, inp)

            def ours(a, lanes=None):
                return lambda: pccl._reduce_scatter(out, inp, group, use_pccl_cpp_backend=True, algorithm=a,
                                                    lanes=lanes)

            wire = n * es                                   # bytes of one block
        ms_nccl = time_something(nccl, warmup_iters=args.warmup, timed_iters=args.iters)
        busbw = lambda ms: (world - 1) * wire / (ms * 1e-3) / 1e9 if world > 1 and ms > 0 else 0.0  # noqa: E731
        rec = {"sweep": sweep, "collective": collective, "P": world, "dtype": str(dtype).replace("torch.", ""),
               "per_rank_bytes": nbytes, "nccl_ms": round(ms_nccl, 5), "nccl_busbw_gbs": round(busbw(ms_nccl), 2),
               "variants": {}}
        names = variants(collective)
        cap = comm.native.eager_capacity
        if args.algorithms == "all" and cap > 0 and (world * nbytes if collective == "all_gather" else (world - 1) * wire) <= cap:
            names = names + [sch.EAGER]
        if len(lane_counts) > 1:
            names = [f"{a}@{n_l}" for a in names for n_l in lane_counts]
        for a in names:
            algo, _, at = a.partition("@")
            fn = ours(algo, int(at) if at else lane_counts[0])
            ms = time_something(fn, warmup_iters=args.warmup, timed_iters=args.iters)
            comm.check()
            good = None
            if args.test:
                nccl()
                out.zero_()
                fn()
                torch.cuda.synchronize()
                if collective == "all_gather":
                    good = torch.equal(out, gold)
                else:
                    # NCCL rounds partial sums in the input dtype; compare with a tolerance that covers it
                    rtol, atol = (1e-5, 1e-5) if dtype == torch.float32 else (4e-2, 4e-2)
                    close = torch.isclose(out.float(), gold.float(), rtol=rtol, atol=atol)
                    good = float((~close).sum()) <= 0.02 * n
                flag = torch.tensor([1 if good else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                good = bool(flag.item())
                ok_all = ok_all and good
            rec["variants"][a] = {"ms": round(ms, 5), "busbw_gbs": round(busbw(ms), 2),
                                  "vs_nccl": round(ms_nccl / ms, 3) if ms > 0 else None, "correct": good}
        plain = {a: v for a, v in rec["variants"].items() if a.partition("@")[0] != sch.MULTIMEM}
        for key, pool in (("best", rec["variants"]), ("best_without_multimem", plain)):
            if pool:
                a = min(pool, key=lambda k: pool[k]["ms"])
                rec[key] = {"variant": a, **pool[a], "frac_of_900": round(pool[a]["busbw_gbs"] / NVLINK_GBS_NOMINAL, 4),
                            "frac_of_measured_770": round(pool[a]["busbw_gbs"] / NVLINK_GBS_MEASURED, 4)}
        rows.append(rec)
        if rank == 0:
            line = " ".join(f"{a}={v['ms'] * 1e3:.1f}us({v['vs_nccl']}x)" for a, v in rec["variants"].items())
            print(f"{sweep:6s} P={world} {nbytes / (1 << 20):9.3f} MiB nccl={ms_nccl * 1e3:.1f}us {line}", flush=True)
        del inp, out, gold

    if rank == 0:
        if args.test:
            print("All tests passed! PCCL outputs match NCCL outputs!" if ok_all else "TEST FAILED: outputs differ from NCCL")
        doc = {"P": world, "nvls": bool(comm.nvls), "transport": comm.transport_name,
               "timing": f"{args.warmup} warm-up + {args.iters} timed calls in one CUDA-event pair, mean, max over ranks",
               "rows": rows}
        if args.json:
            Path(args.json).parent.mkdir(parents=True, exist_ok=True)
            Path(args.json).write_text(json.dumps(doc, indent=1))
        if args.md:
            Path(args.md).parent.mkdir(parents=True, exist_ok=True)
            Path(args.md).write_text(markdown(doc))
        if args.write_tuning_table:
            for collective, sweep in (("all_gather", "ag"), ("reduce_scatter", "rs")):
                pts = [r for r in rows if r["sweep"] == sweep]
                if pts:
                    update_tuning_table(Path(args.write_tuning_table), collective, world, pts)
    dist.barrier()
    pccl.shutdown()
    dist.destroy_process_group()
    if args.test and not ok_all:
        raise SystemExit(1)


def markdown(doc: Dict) -> str:
    """One table per sweep: time of every variant, NCCL, the winners and their fraction of the link."""
    out = [f"P = {doc['P']}, NVLS {'on' if doc['nvls'] else 'off'}, transport {doc['transport']}; {doc['timing']}.", ""]
    by_sweep: Dict[str, List[Dict]] = {}
    for r in doc["rows"]:
        by_sweep.setdefault(r["sweep"], []).append(r)
    for sweep, rs in by_sweep.items():
        names = []
        for r in rs:                                     # some variants (eager) only exist at small sizes
            names += [a for a in r["variants"] if a not in names]
        out.append(f"### {sweep} ({rs[0]['collective']}, {rs[0]['dtype']})")
        out.append("")
        out.append("| per-rank MiB | NCCL µs | NCCL GB/s | " + " | ".join(f"{a} µs" for a in names) +
                   " | best | GB/s | x NCCL | of 900 | best w/o multimem | GB/s | x NCCL |")
        out.append("|" + "---|" * (len(names) + 10))
        for r in rs:
            b, p = r.get("best", {}), r.get("best_without_multimem", {})
            cells = [f"{r['per_rank_bytes'] / (1 << 20):g}", f"{r['nccl_ms'] * 1e3:.1f}", f"{r['nccl_busbw_gbs']:.1f}"]
            cells += [(f"{r['variants'][a]['ms'] * 1e3:.1f}" + ("" if r['variants'][a]['correct'] in (None, True) else " (WRONG)"))
                      if a in r["variants"] else "-" for a in names]
            cells += [b.get("variant", "-"), f"{b.get('busbw_gbs', 0):.1f}", f"{b.get('vs_nccl', 0)}", f"{b.get('frac_of_900', 0):.2f}",
                      p.get("variant", "-"), f"{p.get('busbw_gbs', 0):.1f}", f"{p.get('vs_nccl', 0)}"]
            out.append("| " + " | ".join(cells) + " |")
        out.append("")
    return "\n".join(out)


if __name__ == "__main__":
    main()
