"""Small, self-terminating workloads for profiler captures (one GPU).

    python benchmark_raw_collectives/profile_cases.py gemm
    python benchmark_raw_collectives/profile_cases.py all_gather      # 8 ranks emulated on one device
    python benchmark_raw_collectives/profile_cases.py reduce_scatter
    python benchmark_raw_collectives/profile_cases.py adamw
    python benchmark_raw_collectives/profile_cases.py cross_entropy

Each case launches its kernel three times on inputs larger than the 126 MB L2 but well
under a few GB, then exits.  Meant to be run plainly first and then under
``ncu --set full --clock-control none -k regex:<kernel> -c 3``.
"""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

import pccl  # noqa: E402
from pccl import schedule as sch  # noqa: E402

DEV = "cuda:0"


def gemm():
    M, N, K = 8192, 6144, 2048
    A = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    W = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        pccl._C.gemm(A, W, None, out)
    torch.cuda.synchronize()


def _emu():
    return pccl.Communicator.emulated_world(8, device=0, heap_bytes=640 << 20, staging_bytes=16 << 20)


def all_gather():
    comm = _emu()
    n = 32 << 20                                    # 32 MiB per rank, 256 MiB gathered per rank
    outs = comm.empty(8 * n, torch.uint8)
    ins = [torch.randint(0, 255, (n,), device=DEV, dtype=torch.uint8) for _ in range(8)]
    for _ in range(3):
        comm.native.all_gather(comm.world_group.gid, outs, ins, sch.ALGO_IDS[sch.DIRECT], 16)
    comm.check()


def reduce_scatter():
    comm = _emu()
    n = 4 << 20                                     # result elements per rank; input 8 * n bf16 = 64 MiB per rank
    sym = comm.empty(8 * n, torch.bfloat16)
    for t in sym:
        t.copy_(torch.randn(8 * n, device=DEV).to(torch.bfloat16))
    outs = [torch.empty(n, device=DEV, dtype=torch.float32) for _ in range(8)]
    for _ in range(3):
        comm.native.reduce_scatter(comm.world_group.gid, outs, sym, sch.ALGO_IDS[sch.PULL], 16, 0.125, None)
    comm.check()


def adamw():
    n = 64 << 20                                    # 64 Mi parameters: 1.3 GB of optimizer traffic per launch
    master = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    grad = torch.randn(n, device=DEV)
    param = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    sq = torch.zeros(1, device=DEV)
    for step in range(1, 4):
        sq.zero_()
        pccl._C.sq_norm(grad, sq)
        pccl._C.adamw(master, m, v, grad, param, 1e-4, 0.9, 0.95, 1e-8, 0.1, step, 1.0, 1.0, sq)
    torch.cuda.synchronize()


def cross_entropy():
    rows, vocab = 4096, 50304                       # 412 MB of bf16 logits
    logits = torch.randn(rows, vocab, device=DEV).to(torch.bfloat16)
    tgt = torch.randint(0, vocab, (rows,), device=DEV)
    loss = torch.zeros(1, device=DEV)
    for _ in range(3):
        pccl._C.ce_fwd_bwd(logits, tgt, loss, 1.0 / rows, -100)
    torch.cuda.synchronize()


if __name__ == "__main__":
    {"gemm": gemm, "all_gather": all_gather, "reduce_scatter": reduce_scatter, "adamw": adamw,
     "cross_entropy": cross_entropy}[sys.argv[1]]()
    print("done", sys.argv[1])
