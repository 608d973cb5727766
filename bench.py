"""Flagship benchmark: ZeRO-3 training step of GPT-1.3B (tokens per second, whole job).

    python bench.py --gpus N --steps K --warmup W            # this library (default arm)
    python bench.py --impl nccl ...                          # same engine over torch.distributed/NCCL
    python bench.py --impl reference ...                     # the unmodified reference, if it can run

For N > 1 start it with torchrun (one process per GPU); RANK / LOCAL_RANK / WORLD_SIZE /
MASTER_* are read from the environment.  Rank 0 prints ONE JSON line.

Configuration (fourth benchmark configuration of the reference's baseline description):
24 layers, d_model 2048, 16 heads, FFN 8192 GELU, vocabulary 50304, sequence 2048,
micro-batch 4 per GPU, bf16 compute with fp32 master weights and Adam moments, random
N(0, 0.02) weights, token ids uniform in [0, 50304).  Weak scaling: per-GPU work is fixed.

Timing: W (>= 3) untimed steps, then exactly K steps between two CUDA events, bracketed
by a barrier and a device synchronisation, maximum over ranks.  A step's working set
(parameters, activations, gradients: tens of GB) is far larger than the 126 MB L2, so no
explicit flush is needed between steps.  A second pass measures the same K steps end to
end through ``Zero3Engine.train_step`` fed from pinned host memory, reading the loss back
to the host every step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "zero3_gpt_tokens_per_sec"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="pccl", choices=["pccl", "nccl", "reference"])
    ap.add_argument("--model", default="gpt-1.3b")
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--algorithm", default="auto")
    ap.add_argument("--lanes", type=int, default=int(os.environ.get("PCCL_TRAIN_LANES", "16")),
                    help="SMs a parameter gather / gradient reduction may occupy while it overlaps the GEMMs")
    ap.add_argument("--nvls", type=int, default=int(os.environ.get("PCCL_ENABLE_NVLS", "0")))
    ap.add_argument("--fused-ag-gemm", type=int, default=int(os.environ.get("PCCL_FUSED_AG_GEMM", "0")))
    ap.add_argument("--gather-ctas", type=int, default=16)
    ap.add_argument("--overlap-wgrad", type=int, default=int(os.environ.get("PCCL_OVERLAP_WGRAD", "0")),
                    help="weight-gradient GEMMs on a second stream beside the memory-bound backward kernels")
    ap.add_argument("--fused-gelu-gemm", type=int, default=int(os.environ.get("PCCL_FUSED_GELU_GEMM", "0")),
                    help="FC1 on the library's tcgen05 GEMM with bias+GELU in the epilogue")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def reference_arm(args) -> None:
    """The reference cannot produce this metric: it contains no model, no training loop and
    no DeepSpeed configuration (only the hook ``pccl/patch_deepspeed.py``), every one of its
    modules imports mpi4py at import time, and neither mpi4py nor DeepSpeed nor an MPI
    implementation is installed or installable offline."""
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        print(json.dumps({
            "impl": "reference",
            "unavailable": "reference has no training script or model and imports mpi4py + deepspeed, "
                           "neither installed nor installable offline (no MPI implementation on the box)",
        }))


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import pccl
    from pccl.models.gpt import PRESETS, GPTConfig
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine, heap_bytes_needed
    from pccl.utils.clocks import ClockSampler
    from pccl.utils.env import init_distributed
    from pccl.utils.timing import max_over_ranks

    rank, world, local = init_distributed()
    assert world == args.gpus or "WORLD_SIZE" not in os.environ, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    warmup = max(3, args.warmup)
    cfg = PRESETS[args.model]
    if args.seq_len:
        cfg = GPTConfig(cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab, args.seq_len, name=cfg.name)
    mb = args.micro_batch or (4 if args.model == "gpt-1.3b" else 2)
    S = cfg.seq_len
    dev = torch.device("cuda", torch.cuda.current_device())

    comm = None
    if args.impl == "pccl":
        heap = heap_bytes_needed(cfg, world, bool(args.fused_ag_gemm)) + (320 << 20)
        comm = pccl.init(heap_bytes=heap, staging_bytes=64 << 20, enable_nvls=bool(args.nvls))
        from pccl.patch_deepspeed import patch_deepspeed

        patch_deepspeed(world, algorithm=args.algorithm, lanes=args.lanes)
    backend = TorchBackend()
    engine = Zero3Engine(cfg, backend, OptimConfig(), device=dev, comm=comm, micro_batch=mb,
                         fused_ag_gemm=(args.impl == "pccl" and bool(args.fused_ag_gemm)), gather_ctas=args.gather_ctas,
                         fused_gelu_gemm=bool(args.fused_gelu_gemm), overlap_wgrad=bool(args.overlap_wgrad))

    total_steps = warmup + args.steps
    gen = torch.Generator(device="cpu").manual_seed(4321 + rank)
    host_tokens = torch.randint(0, cfg.vocab, (total_steps, mb, S + 1), generator=gen, dtype=torch.int64).pin_memory()
    dev_tokens = host_tokens.to(dev)

    def step_device(i):
        return engine.train_step(dev_tokens[i, :, :S], dev_tokens[i, :, 1:])

    def step_host(i):
        loss = engine.train_step(host_tokens[i, :, :S], host_tokens[i, :, 1:])
        return float(loss.item())                       # device -> host read of the result

    for i in range(warmup):
        step_device(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.05).start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    launches = 0
    loss = None
    for i in range(args.steps):
        loss = step_device(warmup + i)
        launches += engine.launches
    t_end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = max_over_ranks(t_start.elapsed_time(t_end) / args.steps)
    tokens_per_step = world * mb * S
    value = tokens_per_step / (ms / 1e3)
    engine.check_errors()                               # raises if any kernel gave up in a bounded wait

    e2e = None
    if not args.no_e2e:
        step_host(0)                                    # host path once, untimed
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(args.steps):
            last = step_host(warmup + i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / args.steps)
        e2e = {
            "value": tokens_per_step / (e2e_ms / 1e3),
            "unit": "tokens/s",
            "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": 2 * mb * S * 8,       # tokens and targets, int64, from pinned memory
            "d2h_bytes_per_step": 4,                    # the fp32 loss
            "last_loss": last,
        }

    if rank == 0:
        flops = cfg.flops_per_token() * mb * S            # per GPU per step
        out = {
            "metric": METRIC,
            "value": value,
            "unit": "tokens/s",
            "impl": args.impl,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic: uniform random token ids, random-init N(0,0.02) weights",
            "config": {
                "model": cfg.name, "layers": cfg.n_layer, "d_model": cfg.d_model, "heads": cfg.n_head,
                "ffn": cfg.d_ff, "vocab": cfg.vocab, "params": cfg.num_params(),
                "global_batch": world * mb, "micro_batch_per_gpu": mb, "seq_len": S,
                "parallelism": f"zero3-dp{world}", "optimizer": "AdamW fp32 master+moments, grad-norm clip 1.0",
                "algorithm": args.algorithm, "lanes": args.lanes, "nvls": bool(args.nvls),
                "fused_ag_gemm": bool(engine.fused_ag_gemm), "fused_gelu_gemm": bool(engine.fused_gelu_gemm),
                "overlap_wgrad": bool(engine.overlap_wgrad),
                "l2": "working set per step (tens of GB) exceeds the 126 MB L2; no explicit flush",
                "transport": comm.transport_name if comm is not None else "nccl",
            },
            "model_tflops_per_gpu": flops / (ms / 1e3) / 1e12,
            "final_loss": float(loss.item()) if loss is not None else None,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"], "power_w_max": clocks.get("power_w_max")},
            "gpu_launches": launches,
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
    if comm is not None:
        pccl.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
