"""Flagship benchmark: ZeRO-3 training step of GPT-1.3B (tokens per second, whole job).

    python bench.py --gpus N --steps K --warmup W            # this library, then the NCCL+cuBLAS arm
    python bench.py --impl nccl ...                          # only: same engine over torch.distributed/NCCL, cuBLAS GEMMs
    python bench.py --impl reference ...                     # the unmodified reference, as far as it can run

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

The default run measures three arms back to back in one process, same steps and warm-up:
the library arm (collectives and element-wise kernels of this repository; plain dense
products on cuBLAS, ``--gemm auto``), the same arm with every dense product on this
repository's tcgen05 GEMM (``native_gemm_arm`` in the JSON line; ``--gemm pccl`` makes it the
main arm) and the baseline arm the reference's NCCL build amounts to (the same engine with its
collectives on ``torch.distributed``/NCCL and every dense product on cuBLAS through
``torch``).  ``vs_baseline`` is library arm / baseline arm; the reference publishes no number
of its own, and what it patches is DeepSpeed's backend (``pccl/patch_deepspeed.py:95-126`` of
the reference), which is what ``pccl.patch_deepspeed`` re-routes here.

The reference itself has no model and no training loop, so ``--impl reference`` cannot produce
tokens/s; it prints the ``unavailable`` line and, as evidence for the other half of the metric,
the times of the UNMODIFIED reference's raw-collective benchmark on this machine
(``baseline/run_reference.py``).  The library arm reports the same two sweeps under
``raw_collectives`` so that the two lines can be compared row by row.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
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
                    help="SMs a gradient reduction (or a kernel-driven parameter gather) may occupy while it overlaps the GEMMs")
    ap.add_argument("--nvls", type=int, default=int(os.environ.get("PCCL_ENABLE_NVLS", "1")),
                    help="bind an NVLS multicast mapping where the machine offers one (the multimem variants win the small sizes)")
    ap.add_argument("--gemm", default=os.environ.get("PCCL_GEMM", "auto"), choices=["auto", "pccl", "cublas"],
                    help="library arm: auto = plain dense products on cuBLAS (measured 7 %% faster per step than the "
                         "repository's tcgen05 GEMM) and the fused products (all-gather+GEMM, GEMM+GELU) on the "
                         "repository's kernel, with one more arm that routes every product through it; "
                         "pccl = every product on the repository's GEMM; cublas = none")
    ap.add_argument("--no-native-gemm-arm", action="store_true",
                    help="with --gemm auto: skip the extra arm that runs every dense product on the repository's GEMM")
    ap.add_argument("--gather", default=os.environ.get("PCCL_GATHER", "copy_engine"), choices=["copy_engine", "kernel"],
                    help="library arm: parameter gathers by the copy engines (no SM used) or by the all-gather kernels")
    ap.add_argument("--fused-ag-gemm", type=int, default=int(os.environ.get("PCCL_FUSED_AG_GEMM", "0")))
    ap.add_argument("--gather-ctas", type=int, default=16)
    ap.add_argument("--overlap-wgrad", type=int, default=int(os.environ.get("PCCL_OVERLAP_WGRAD", "0")),
                    help="weight-gradient GEMMs on a second stream beside the memory-bound backward kernels")
    ap.add_argument("--fused-gelu-gemm", type=int, default=int(os.environ.get("PCCL_FUSED_GELU_GEMM", "0")),
                    help="FC1 on the library's tcgen05 GEMM with bias+GELU in the epilogue")
    ap.add_argument("--fused-gelu-bwd", type=int, default=int(os.environ.get("PCCL_FUSED_GELU_BWD", "0")),
                    help="GELU backward as the epilogue of the data-gradient GEMM in front of it (library GEMM only)")
    ap.add_argument("--dynamic-tiles", type=int, default=int(os.environ.get("PCCL_DYNAMIC_TILES", "-1")),
                    help="library GEMM hands tiles out at run time: 1 on, 0 off, -1 on when N > 1")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baseline", action="store_true", help="library arm only: skip the NCCL+cuBLAS arm and vs_baseline")
    ap.add_argument("--no-raw", action="store_true", help="skip the raw-collective rows")
    return ap.parse_args()


# ------------------------------------------------------------------------------------ reference arm
def reference_arm(args) -> None:
    """The reference cannot produce tokens/s: it contains no model, no training loop and no
    DeepSpeed configuration (only the hook ``pccl/patch_deepspeed.py``), and DeepSpeed is neither
    installed nor installable offline.  What it can run is its raw-collective benchmark on its
    NCCL branch; every rank starts that as a child process (the unmodified scripts create and
    destroy their own process group) and rank 0 attaches the rows."""
    rank = int(os.environ.get("RANK", "0"))
    out = {
        "impl": "reference",
        "unavailable": "reference has no training script or model (its DeepSpeed hook expects an external GPT script) "
                       "and DeepSpeed is not installable offline: tokens/s cannot be produced by it; its raw-collective "
                       "benchmark (NCCL branch, unmodified, behind an import stand-in for mpi4py) is attached",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
    }
    raw = {}
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    for i, kind in enumerate(("all_gather", "reduce_scatter")):
        env = dict(os.environ)
        # a process group of its own per child: its own rendezvous port, not torchrun's agent store
        env["MASTER_ADDR"] = env.get("MASTER_ADDR", "127.0.0.1")
        env["MASTER_PORT"] = str(base_port + 7 + i)
        env.pop("TORCHELASTIC_USE_AGENT_STORE", None)
        with tempfile.TemporaryDirectory() as td:
            jp = os.path.join(td, f"{kind}.json")
            try:
                r = subprocess.run([sys.executable, str(ROOT / "baseline" / "run_reference.py"), kind, "--json", jp],
                                   env=env, capture_output=True, text=True, timeout=900)
                if rank == 0:
                    if r.returncode == 0 and os.path.exists(jp):
                        raw[kind] = json.loads(Path(jp).read_text())
                    else:
                        raw[kind] = {"unavailable": f"exit code {r.returncode}: {(r.stderr or r.stdout)[-300:]}"}
            except subprocess.TimeoutExpired:
                if rank == 0:
                    raw[kind] = {"unavailable": "timed out after 900 s"}
    if rank == 0:
        out["raw_collectives"] = raw
        print(json.dumps(out))


# ------------------------------------------------------------------------------------ measured arms
def run_arm(args, impl: str, ctx: dict, native_gemm: bool = False, e2e: bool = True) -> dict:
    """One arm: build the engine, warm up, time K steps on the device, then K steps end to end."""
    import torch
    import torch.distributed as dist

    import pccl
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine, heap_bytes_needed
    from pccl.patch_deepspeed import patch_deepspeed, unpatch_deepspeed
    from pccl.utils.clocks import ClockSampler
    from pccl.utils.timing import max_over_ranks

    rank, world, cfg, mb, S, dev = ctx["rank"], ctx["world"], ctx["cfg"], ctx["mb"], ctx["S"], ctx["dev"]
    warmup = ctx["warmup"]
    comm = None
    library = impl == "pccl"
    if library:
        if ctx.get("comm") is None:
            heap = heap_bytes_needed(cfg, world, bool(args.fused_ag_gemm)) + (320 << 20)
            if not args.no_raw:
                heap += 2304 << 20          # the 1 GiB points of the two raw-collective sweeps: output + input, or input
            ctx["comm"] = pccl.init(heap_bytes=heap, staging_bytes=64 << 20, enable_nvls=bool(args.nvls))
        comm = ctx["comm"]
        patch_deepspeed(world, algorithm=args.algorithm, lanes=args.lanes)
    else:
        unpatch_deepspeed()
    engine = Zero3Engine(cfg, TorchBackend(), OptimConfig(), device=dev, comm=comm, micro_batch=mb,
                         fused_ag_gemm=(library and bool(args.fused_ag_gemm)), gather_ctas=args.gather_ctas,
                         fused_gelu_gemm=(library and bool(args.fused_gelu_gemm)), overlap_wgrad=bool(args.overlap_wgrad),
                         native_gemm=(library and native_gemm), fused_gelu_bwd_gemm=bool(args.fused_gelu_bwd),
                         dynamic_tiles=None if args.dynamic_tiles < 0 else bool(args.dynamic_tiles),
                         copy_engine_gather=(library and args.gather == "copy_engine"))
    host_tokens, dev_tokens = ctx["host_tokens"], ctx["dev_tokens"]

    def step_device(i):
        return engine.train_step(dev_tokens[i, :, :S], dev_tokens[i, :, 1:])

    def step_host(i):
        loss = engine.train_step(host_tokens[i, :, :S], host_tokens[i, :, 1:])
        return float(loss.item())                       # device -> host read of the result

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(warmup):
        step_device(i)
    fence()
    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.05).start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    launches = 0
    loss = None
    for i in range(args.steps):
        loss = step_device(warmup + i)
        launches += engine.launches
    t_end.record()
    fence()
    clocks = sampler.stop()
    ms = max_over_ranks(t_start.elapsed_time(t_end) / args.steps)
    tokens_per_step = world * mb * S
    engine.check_errors()                               # raises if any kernel gave up in a bounded wait
    res = {
        "impl": impl, "value": tokens_per_step / (ms / 1e3), "ms_per_step": ms,
        "final_loss": float(loss.item()) if loss is not None else None,
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                   "samples": clocks["samples"], "power_w_max": clocks.get("power_w_max")},
        "gpu_launches": launches,
        "engine": {"fused_ag_gemm": bool(engine.fused_ag_gemm), "fused_gelu_gemm": bool(engine.fused_gelu_gemm),
                   "overlap_wgrad": bool(engine.overlap_wgrad), "native_gemm": bool(engine.native_gemm),
                   "fused_gelu_bwd_gemm": bool(engine.fused_gelu_bwd_gemm), "dynamic_tiles": bool(engine.dynamic_tiles),
                   "copy_engine_gather": bool(engine.copy_engine_gather)},
    }
    if e2e and not args.no_e2e:
        step_host(0)                                    # host path once, untimed
        fence()
        t0 = time.perf_counter()
        last = None
        for i in range(args.steps):
            last = step_host(warmup + i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / args.steps)
        res["e2e"] = {
            "value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": 2 * mb * S * 8,       # tokens and targets, int64, from pinned memory
            "d2h_bytes_per_step": 4,                    # the fp32 loss
            "last_loss": last,
        }
        engine.check_errors()
    del engine
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return res


def raw_collectives(ctx: dict) -> dict:
    """The reference's two sweeps (all-gather: total output 1..1024 MiB, bf16; reduce-scatter: total
    input 1..1024 MiB, fp32) through this library's public calls with ``algorithm="auto"``, timed
    the way the reference times (5 warm-up + 20 calls in one CUDA-event pair), max over ranks."""
    import torch

    import pccl
    from pccl.utils.timing import time_something

    world, rank, dev, comm = ctx["world"], ctx["rank"], ctx["dev"], ctx["comm"]
    out = {"all_gather": {"dtype": "bf16", "size_mode": "total_output", "rows": []},
           "reduce_scatter": {"dtype": "fp32", "size_mode": "total_input", "rows": []},
           "timing": "5 warm-up + 20 timed calls, one CUDA-event pair, mean, max over ranks; algorithm=auto"}
    free = comm.native.heap_bytes - comm.native.heap_used - (8 << 20)
    for mib in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024):
        total = mib << 20
        if total + total // world + (1 << 20) <= free:
            n = total // 2 // world
            inp, o = comm.empty(n, torch.bfloat16), comm.empty(n * world, torch.bfloat16)
            inp.normal_()
            ms = time_something(lambda: pccl.all_gather(o, inp), warmup_iters=5, timed_iters=20)
            out["all_gather"]["rows"].append({"size_mib": mib, "time_ms": ms})
            del inp, o
        if total + (1 << 20) <= free:
            n = total // 4 // world
            inp, o = comm.empty(n * world, torch.float32), torch.empty(n, dtype=torch.float32, device=dev)
            inp.normal_()
            ms = time_something(lambda: pccl.reduce_scatter(o, inp), warmup_iters=5, timed_iters=20)
            out["reduce_scatter"]["rows"].append({"size_mib": mib, "time_ms": ms})
            del inp, o
    comm.check()
    return out


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import pccl
    from pccl.models.gpt import PRESETS, GPTConfig
    from pccl.utils.env import init_distributed

    rank, world, local = init_distributed()
    assert world == args.gpus or "WORLD_SIZE" not in os.environ, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    warmup = max(3, args.warmup)
    cfg = PRESETS[args.model]
    if args.seq_len:
        cfg = GPTConfig(cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab, args.seq_len, name=cfg.name)
    mb = args.micro_batch or (4 if args.model == "gpt-1.3b" else 2)
    S = cfg.seq_len
    dev = torch.device("cuda", torch.cuda.current_device())
    total_steps = warmup + args.steps
    gen = torch.Generator(device="cpu").manual_seed(4321 + rank)
    host_tokens = torch.randint(0, cfg.vocab, (total_steps, mb, S + 1), generator=gen, dtype=torch.int64).pin_memory()
    ctx = {"rank": rank, "world": world, "cfg": cfg, "mb": mb, "S": S, "dev": dev, "warmup": warmup,
           "host_tokens": host_tokens, "dev_tokens": host_tokens.to(dev), "comm": None}

    main_arm = run_arm(args, args.impl, ctx, native_gemm=(args.gemm == "pccl"))
    native_arm = None
    if args.impl == "pccl" and args.gemm == "auto" and not args.no_native_gemm_arm:
        native_arm = run_arm(args, "pccl", ctx, native_gemm=True, e2e=False)
    base_arm = None
    if args.impl == "pccl" and not args.no_baseline:
        base_arm = run_arm(args, "nccl", ctx)
    raw = None
    if args.impl == "pccl" and not args.no_raw and ctx["comm"] is not None:
        raw = raw_collectives(ctx)

    if rank == 0:
        flops = cfg.flops_per_token() * mb * S            # per GPU per step
        ms = main_arm["ms_per_step"]
        comm = ctx["comm"]
        out = {
            "metric": METRIC,
            "value": main_arm["value"],
            "unit": "tokens/s",
            "impl": args.impl,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": (main_arm["value"] / base_arm["value"]) if base_arm else None,
            "dtype": "bf16",
            "data": "synthetic: uniform random token ids, random-init N(0,0.02) weights",
            "config": {
                "model": cfg.name, "layers": cfg.n_layer, "d_model": cfg.d_model, "heads": cfg.n_head,
                "ffn": cfg.d_ff, "vocab": cfg.vocab, "params": cfg.num_params(),
                "global_batch": world * mb, "micro_batch_per_gpu": mb, "seq_len": S,
                "parallelism": f"zero3-dp{world}", "optimizer": "AdamW fp32 master+moments, grad-norm clip 1.0",
                "algorithm": args.algorithm, "lanes": args.lanes, "nvls": bool(args.nvls),
                "gemm": "tcgen05 (this repository)" if main_arm["engine"]["native_gemm"] else
                        ("cuBLAS for the plain products, tcgen05 (this repository) for the fused ones that are switched on"
                         if args.impl == "pccl" and args.gemm == "auto" else "cuBLAS"),
                "parameter_gather": "copy engines" if main_arm["engine"]["copy_engine_gather"] else
                                    ("all-gather kernels" if args.impl == "pccl" and world > 1 else "nccl" if world > 1 else "none (one rank)"),
                **{k: v for k, v in main_arm["engine"].items() if k in ("fused_ag_gemm", "fused_gelu_gemm", "fused_gelu_bwd_gemm", "overlap_wgrad", "dynamic_tiles")},
                "l2": "working set per step (tens of GB) exceeds the 126 MB L2; no explicit flush",
                "transport": comm.transport_name if (comm is not None and args.impl == "pccl") else "nccl",
            },
            "model_tflops_per_gpu": flops / (ms / 1e3) / 1e12,
            "final_loss": main_arm["final_loss"],
            "clocks": main_arm["clocks"],
            "gpu_launches": main_arm["gpu_launches"],
        }
        if "e2e" in main_arm:
            out["e2e"] = main_arm["e2e"]
        if base_arm is not None:
            out["baseline_arm"] = {
                "what": "same engine, collectives on torch.distributed/NCCL, dense products on cuBLAS: what the "
                        "reference's NCCL build amounts to (the reference has no model of its own)",
                "value": base_arm["value"], "ms_per_step": base_arm["ms_per_step"], "clocks": base_arm["clocks"],
                "e2e_value": base_arm.get("e2e", {}).get("value"), "final_loss": base_arm["final_loss"],
            }
            if "e2e" in main_arm and "e2e" in base_arm:
                out["e2e"]["vs_baseline"] = main_arm["e2e"]["value"] / base_arm["e2e"]["value"]
        if native_arm is not None:
            out["native_gemm_arm"] = {
                "what": "the same library arm with every dense product (forward, data and weight gradients) on the "
                        "repository's tcgen05 GEMM instead of cuBLAS",
                "value": native_arm["value"], "ms_per_step": native_arm["ms_per_step"], "clocks": native_arm["clocks"],
                "gpu_launches": native_arm["gpu_launches"], "final_loss": native_arm["final_loss"],
                "vs_baseline": (native_arm["value"] / base_arm["value"]) if base_arm else None,
            }
        if raw is not None:
            out["raw_collectives"] = raw
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
    if ctx["comm"] is not None:
        pccl.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
