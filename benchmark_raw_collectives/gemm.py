"""Throughput of the tcgen05 GEMM (and of the fused all-gather+GEMM) against cuBLAS.

    python benchmark_raw_collectives/gemm.py                       # one GPU: tcgen05 vs torch.matmul
    python benchmark_raw_collectives/gemm.py --layouts nt,nn,tn    # forward, data-gradient and weight-gradient forms
    torchrun --nproc-per-node 8 benchmark_raw_collectives/gemm.py --fused --gather-ctas 16
    torchrun --nproc-per-node 8 benchmark_raw_collectives/gemm.py --fused --copy-engine

Shapes are the GEMMs that consume freshly gathered weights in the two benchmark models
(QKV and FC1 of GPT-1.3B with 8192 tokens per GPU, of GPT-7B with 4096 tokens per GPU) plus
a square 8192.  Every call is timed by its own CUDA-event pair after an L2 flush (the
operands are smaller than the 126 MB L2), median over the timed calls, maximum over ranks.
The fused mode compares ONE kernel (gather + multiply) with the baseline sequence
NCCL all_gather_into_tensor followed by torch.matmul.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from pccl.utils.env import init_distributed  # noqa: E402
from pccl.utils.timing import flush_l2, max_over_ranks  # noqa: E402

SHAPES = {
    "1.3b-qkv": (8192, 6144, 2048),
    "1.3b-fc1": (8192, 8192, 2048),
    "7b-qkv": (4096, 12288, 4096),
    "7b-fc1": (4096, 16384, 4096),
    "square-8k": (8192, 8192, 8192),
}

# Every dense product of one GPT-1.3B training step with 8192 tokens per GPU, as (layout, M, N, K, count
# per step): forward x W^T (nt), data gradients dy W (nn), weight gradients dy^T x (tn), and the head.
STEP_1P3B = [
    ("nt", 8192, 6144, 2048, 24), ("nt", 8192, 2048, 2048, 24), ("nt", 8192, 8192, 2048, 24), ("nt", 8192, 2048, 8192, 24),
    ("nn", 8192, 8192, 2048, 24), ("nn", 8192, 2048, 8192, 24), ("nn", 8192, 2048, 2048, 24), ("nn", 8192, 2048, 6144, 24),
    ("tn", 2048, 8192, 8192, 24), ("tn", 8192, 2048, 8192, 24), ("tn", 2048, 2048, 8192, 24), ("tn", 6144, 2048, 8192, 24),
    ("nt", 8192, 50304, 2048, 1), ("nn", 8192, 2048, 50304, 1), ("tn", 50304, 2048, 8192, 1),
]


def operands(layout, M, N, K, dev, g):
    """(ours, ref, out) closures for C[M,N] = sum_k a[m,k] b[n,k] with the operands stored as `layout` says."""
    import pccl

    A = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    W = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    if layout == "nt":
        return (lambda: pccl._C.gemm_ex(A, W, False, False, None, out)), (lambda: torch.matmul(A, W.t(), out=out)), out
    if layout == "nn":
        Wt = W.t().contiguous()                       # stored [K, N]
        del W
        return (lambda: pccl._C.gemm_ex(A, Wt, False, True, None, out)), (lambda: torch.matmul(A, Wt, out=out)), out
    if layout == "tn":
        At, Wt = A.t().contiguous(), W.t().contiguous()   # stored [K, M] and [K, N]
        del A, W
        return (lambda: pccl._C.gemm_ex(At, Wt, True, True, None, out)), (lambda: torch.matmul(At.t(), Wt, out=out)), out
    raise SystemExit(f"unknown layout {layout!r}")


def sustained(fn, seconds=0.25):
    """Mean ms per call of back-to-back calls for about `seconds`: the rate under the power cap,
    which is what a kernel sees inside a long training step (operands stay in L2 where they fit)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    e.synchronize()
    n = max(5, int(seconds * 1e3 / max(s.elapsed_time(e), 1e-3)))
    s.record()
    for _ in range(n):
        fn()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / n


def step_table(args, dev, rank, peak):
    """Per-shape times of a training step's products: this library against cuBLAS, isolated
    (L2 flushed, median) and sustained (back to back), plus the step totals."""
    g = torch.Generator(device=dev).manual_seed(3)
    rows, tot = [], {"ours_ms": 0.0, "cublas_ms": 0.0, "ours_sus_ms": 0.0, "cublas_sus_ms": 0.0}
    for layout, M, N, K, count in STEP_1P3B:
        ours, ref, _out = operands(layout, M, N, K, dev, g)
        ms_o, ms_r = timed(ours, iters=args.iters), timed(ref, iters=args.iters)
        su_o, su_r = sustained(ours), sustained(ref)
        flops = 2.0 * M * N * K
        row = {"layout": layout, "M": M, "N": N, "K": K, "count": count, "tcgen05_ms": ms_o, "cublas_ms": ms_r,
               "vs_cublas": ms_r / ms_o, "tcgen05_sustained_ms": su_o, "cublas_sustained_ms": su_r,
               "vs_cublas_sustained": su_r / su_o, "tcgen05_tflops": flops / ms_o / 1e9,
               "tcgen05_sustained_tflops": flops / su_o / 1e9}
        rows.append(row)
        tot["ours_ms"] += count * ms_o
        tot["cublas_ms"] += count * ms_r
        tot["ours_sus_ms"] += count * su_o
        tot["cublas_sus_ms"] += count * su_r
        if rank == 0:
            print(json.dumps(row), flush=True)
        del ours, ref, _out
    if rank == 0:
        print(json.dumps({"step_totals_ms": tot}), flush=True)
    return rows + [{"step_totals_ms": tot}]


def timed(fn, warmup=3, iters=20):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        ts.append(s.elapsed_time(e))
    return max_over_ranks(statistics.median(ts))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fused", action="store_true")
    ap.add_argument("--gather-ctas", type=int, default=16)
    ap.add_argument("--shapes", default=",".join(SHAPES))
    ap.add_argument("--one-sm", action="store_true", help="use the one-CTA-per-tile form instead of CTA pairs")
    ap.add_argument("--copy-engine", action="store_true",
                    help="fused mode: the copy engines gather (no gatherer CTAs, every SM multiplies)")
    ap.add_argument("--panels-per-copy", type=int, default=0, help="copy-engine gather: 256-row panels per copy (0: a whole shard)")
    ap.add_argument("--layouts", default="nt", help="plain mode: comma list of nt (x W^T), nn (dy W), tn (dy^T x)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--step-shapes", action="store_true",
                    help="time every dense product of a GPT-1.3B training step (all three layouts) against cuBLAS")
    ap.add_argument("--wide", type=int, default=-1,
                    help="plain CTA-pair products in units of two row-tiles that share their W half: 1 always, 0 never, "
                         "-1 where it was measured faster (gemm_set_wide)")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world, _ = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    import pccl
    pccl._C.gemm_set_wide(args.wide)
    from pccl.ops.ag_gemm import AllGatherLinear, auto_gather_ctas

    peaks = {}
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        peaks = json.loads(p.read_text())
    peak = peaks.get("bf16_tflops", 1590.0)
    rows = []
    comm = None
    from pccl.utils.clocks import ClockSampler

    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.05).start()
    if args.fused:
        comm = pccl.init(heap_bytes=1 << 30, staging_bytes=16 << 20)
    if args.step_shapes:
        rows = step_table(args, dev, rank, peak)
    for name in ([] if args.step_shapes else args.shapes.split(",")):
        M, N, K = SHAPES[name]
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        A = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        flops = 2.0 * M * N * K
        if not args.fused:
            for layout in args.layouts.split(","):
                # the same product C[M,N] = sum_k a[m,k] b[n,k], with the operands stored as the layout says
                W = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
                if layout == "nt":
                    ours = lambda: pccl._C.gemm(A, W, None, out, not args.one_sm)  # noqa: E731
                    ref = lambda: torch.matmul(A, W.t(), out=out)  # noqa: E731
                elif layout == "nn":
                    Wt = W.t().contiguous()                       # stored [K, N]
                    ours = lambda: pccl._C.gemm_ex(A, Wt, False, True, None, out)  # noqa: E731
                    ref = lambda: torch.matmul(A, Wt, out=out)  # noqa: E731
                elif layout == "tn":
                    At, Wt = A.t().contiguous(), W.t().contiguous()   # stored [K, M] and [K, N]
                    ours = lambda: pccl._C.gemm_ex(At, Wt, True, True, None, out)  # noqa: E731
                    ref = lambda: torch.matmul(At.t(), Wt, out=out)  # noqa: E731
                else:
                    raise SystemExit(f"unknown layout {layout!r}")
                ms_ours = timed(ours, iters=args.iters)
                ms_ref = timed(ref, iters=args.iters)
                ours()
                y = out.clone()
                ref()
                torch.cuda.synchronize()
                ok = int(pccl._C.gemm_error_word(torch.cuda.current_device()).item()) == 0 and \
                    float((y.float() - out.float()).abs().max()) < 0.25
                row = {"shape": name, "layout": layout, "M": M, "N": N, "K": K, "tcgen05_ms": ms_ours, "cublas_ms": ms_ref,
                       "tcgen05_tflops": flops / ms_ours / 1e9, "cublas_tflops": flops / ms_ref / 1e9,
                       "vs_cublas": ms_ref / ms_ours, "frac_of_measured_peak": flops / ms_ours / 1e9 / peak,
                       "cta_pair": not args.one_sm, "correct": ok}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            continue
        else:
            if N % (world * 256) != 0:
                continue
            lin = AllGatherLinear(comm, None, N, K, gather_ctas=args.gather_ctas, two_cta=not args.one_sm,
                                  copy_engine=args.copy_engine, panels_per_copy=args.panels_per_copy)
            lin.w_shard.copy_((torch.randn(N // world, K, device=dev, generator=g) * 0.02).to(torch.bfloat16))
            torch.cuda.synchronize()
            dist.barrier()
            w_gold = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def baseline():
                dist.all_gather_into_tensor(w_gold, lin.w_shard)
                torch.matmul(A, w_gold.t(), out=out)

            ms_ref = timed(baseline, iters=args.iters)
            ms_ours = timed(lambda: lin(A), iters=args.iters)
            y = lin(A, check=True)
            baseline()
            torch.cuda.synchronize()
            ok = torch.equal(lin.w_full, w_gold) and float((y.float() - out.float()).abs().max()) < 0.25
            remote = (world - 1) / world * N * K * 2
            t_math = flops / (peak * 1e12) * 1e3
            t_link = remote / 770e9 * 1e3
            row = {"shape": name, "M": M, "N": N, "K": K, "P": world, "fused_ms": ms_ours, "nccl_plus_cublas_ms": ms_ref,
                   "roofline_ms": max(t_math, t_link), "frac_of_roofline": max(t_math, t_link) / ms_ours,
                   "speedup_vs_baseline": ms_ref / ms_ours,
                   "gather": "copy engines" if args.copy_engine else "gatherer CTAs",
                   "gather_ctas": 0 if args.copy_engine else (args.gather_ctas if args.gather_ctas > 0 else auto_gather_ctas(M, N, K, world)),
                   "cta_pair": not args.one_sm, "correct": bool(ok)}
            del lin
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    clocks = sampler.stop()
    if rank == 0:
        print(json.dumps({"clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons", "samples", "power_w_max")}}), flush=True)
    if args.json and rank == 0:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps({"rows": rows, "clocks": clocks}, indent=1, default=str))
    if dist.is_initialized():
        dist.barrier()
        if comm is not None:
            pccl.shutdown()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
