"""Throughput of the tcgen05 GEMM (and of the fused all-gather+GEMM) against cuBLAS.

    python benchmark_raw_collectives/gemm.py                       # one GPU: tcgen05 vs torch.matmul
    torchrun --nproc-per-node 8 benchmark_raw_collectives/gemm.py --fused --gather-ctas 16

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


def timed(fn, warmup=3, iters=10):
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
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world, _ = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    import pccl
    from pccl.ops.ag_gemm import AllGatherLinear, auto_gather_ctas

    peaks = {}
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        peaks = json.loads(p.read_text())
    peak = peaks.get("bf16_tflops", 1590.0)
    rows = []
    comm = None
    if args.fused:
        comm = pccl.init(heap_bytes=1 << 30, staging_bytes=16 << 20)
    for name in args.shapes.split(","):
        M, N, K = SHAPES[name]
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        A = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        flops = 2.0 * M * N * K
        if not args.fused:
            W = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            ms_ours = timed(lambda: pccl._C.gemm(A, W, None, out, not args.one_sm))
            ms_ref = timed(lambda: torch.matmul(A, W.t(), out=out))
            y, err = pccl._C.gemm(A, W, None, None, not args.one_sm)
            ok = int(err.item()) == 0 and float((y.float() - (A.float() @ W.float().t())).abs().max()) < 0.5
            row = {"shape": name, "M": M, "N": N, "K": K, "tcgen05_ms": ms_ours, "cublas_ms": ms_ref,
                   "tcgen05_tflops": flops / ms_ours / 1e9, "cublas_tflops": flops / ms_ref / 1e9,
                   "frac_of_measured_peak": flops / ms_ours / 1e9 / peak, "cta_pair": not args.one_sm, "correct": ok}
        else:
            if N % (world * 256) != 0:
                continue
            lin = AllGatherLinear(comm, None, N, K, gather_ctas=args.gather_ctas, two_cta=not args.one_sm)
            lin.w_shard.copy_((torch.randn(N // world, K, device=dev, generator=g) * 0.02).to(torch.bfloat16))
            torch.cuda.synchronize()
            dist.barrier()
            w_gold = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def baseline():
                dist.all_gather_into_tensor(w_gold, lin.w_shard)
                torch.matmul(A, w_gold.t(), out=out)

            ms_ref = timed(baseline)
            ms_ours = timed(lambda: lin(A))
            y = lin(A, check=True)
            baseline()
            torch.cuda.synchronize()
            ok = torch.equal(lin.w_full, w_gold) and float((y.float() - out.float()).abs().max()) < 0.25
            remote = (world - 1) / world * N * K * 2
            t_math = flops / (peak * 1e12) * 1e3
            t_link = remote / 770e9 * 1e3
            row = {"shape": name, "M": M, "N": N, "K": K, "P": world, "fused_ms": ms_ours, "nccl_plus_cublas_ms": ms_ref,
                   "roofline_ms": max(t_math, t_link), "frac_of_roofline": max(t_math, t_link) / ms_ours,
                   "speedup_vs_baseline": ms_ref / ms_ours, "gather_ctas": args.gather_ctas if args.gather_ctas > 0 else auto_gather_ctas(M, N, K, world),
                   "cta_pair": not args.one_sm, "correct": bool(ok)}
            del lin
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if args.json and rank == 0:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))
    if dist.is_initialized():
        dist.barrier()
        if comm is not None:
            pccl.shutdown()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
