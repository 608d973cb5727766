"""Small, self-terminating workloads for profiler captures (one GPU).

    python benchmark_raw_collectives/profile_cases.py gemm
    python benchmark_raw_collectives/profile_cases.py all_gather      # 8 ranks emulated on one device
    python benchmark_raw_collectives/profile_cases.py reduce_scatter
    python benchmark_raw_collectives/profile_cases.py adamw
    python benchmark_raw_collectives/profile_cases.py cross_entropy
    python benchmark_raw_collectives/profile_cases.py gemm_nn | gemm_tn | gemm_split | cublas_gemm
    python benchmark_raw_collectives/profile_cases.py all_gather_ring | all_gather_recursive
    python benchmark_raw_collectives/profile_cases.py reduce_scatter_ring | reduce_scatter_recursive
    python benchmark_raw_collectives/profile_cases.py all_reduce | all_reduce_ring | broadcast
    python benchmark_raw_collectives/profile_cases.py layer_norm | gelu | col_sum

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


def cublas_gemm():
    """The library kernel on the same product, for a side-by-side reading of the counters."""
    M, N, K = 8192, 6144, 2048
    A = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    W = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        torch.matmul(A, W.t(), out=out)
    torch.cuda.synchronize()


def gemm_proj(cublas: bool = False):
    """The output projection of an attention block, 8192 x 2048 out of K = 2048: a short contraction whose
    operands and result (75 MB) stay in L2 between launches, as inside a training step."""
    M, N, K = 8192, 2048, 2048
    A = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    W = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(4):
        if cublas:
            torch.matmul(A, W.t(), out=out)
        else:
            pccl._C.gemm_ex(A, W, False, False, None, out)
    torch.cuda.synchronize()


def gemm_wide():
    """Units of two row-tiles that share their W half: the data gradient 8192 x 2048 out of K = 8192."""
    M, N, K = 8192, 2048, 8192
    dy = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    W = (torch.randn(K, N, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    pccl._C.gemm_set_wide(1)
    for _ in range(3):
        pccl._C.gemm_ex(dy, W, False, True, None, out)
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


def gemm_nn():
    """Data gradient dy @ W: 8192 x 2048 out of K = 8192, second operand read as stored [K, N]."""
    M, N, K = 8192, 2048, 8192
    dy = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    W = (torch.randn(K, N, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        pccl._C.gemm_ex(dy, W, False, True, None, out)
    torch.cuda.synchronize()


def gemm_tn():
    """Weight gradient dy^T @ x: 8192 x 2048 out of 8192 tokens, both operands read as stored."""
    M, N, K = 8192, 2048, 8192
    dy = torch.randn(K, M, device=DEV).to(torch.bfloat16)
    x = torch.randn(K, N, device=DEV).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        pccl._C.gemm_ex(dy, x, True, True, None, out)
    torch.cuda.synchronize()


def gemm_split():
    """64 tiles on 74 CTA pairs: every tile is split along K and finished from fp32 partial sums."""
    M, N, K = 2048, 2048, 8192
    A = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    W = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, device=DEV, dtype=torch.uint8)
    pccl._C.gemm_set_split_last_wave(True, True)     # fewer tiles than CTA pairs: the split is opt-in for those
    for _ in range(3):
        flush.zero_()                                # operands are smaller than L2: start every launch cold
        pccl._C.gemm_ex(A, W, False, False, None, None)
    torch.cuda.synchronize()


def _ag(algo):
    comm = _emu()
    n = 32 << 20
    outs = comm.empty(8 * n, torch.uint8)
    ins = [torch.randint(0, 255, (n,), device=DEV, dtype=torch.uint8) for _ in range(8)]
    for _ in range(3):
        comm.native.all_gather(comm.world_group.gid, outs, ins, sch.ALGO_IDS[algo], 16)
    comm.check()


def _rs(algo):
    comm = pccl.Communicator.emulated_world(8, device=0, heap_bytes=640 << 20, staging_bytes=64 << 20)
    n = 4 << 20
    ins = [torch.randn(8 * n, device=DEV).to(torch.bfloat16) for _ in range(8)]
    outs = [torch.empty(n, device=DEV, dtype=torch.float32) for _ in range(8)]
    for _ in range(3):
        comm.native.reduce_scatter(comm.world_group.gid, outs, ins, sch.ALGO_IDS[algo], 16, 0.125, None)
    comm.check()


def _ar(algo):
    comm = pccl.Communicator.emulated_world(8, device=0, heap_bytes=640 << 20, staging_bytes=64 << 20)
    n = 32 << 20                                    # 64 MiB of bf16 per rank
    sym = comm.empty(n, torch.bfloat16)
    for t in sym:
        t.copy_(torch.randn(n, device=DEV).to(torch.bfloat16))
    for _ in range(3):
        comm.native.all_reduce(comm.world_group.gid, sym, sch.ALGO_IDS[algo], 16, 1.0)
    comm.check()


def broadcast():
    comm = _emu()
    n = 32 << 20
    sym = comm.empty(n, torch.uint8)
    for _ in range(3):
        comm.native.broadcast(comm.world_group.gid, sym, 0, 16, False)
    comm.check()


def layer_norm():
    """Residual add + layer norm forward, and the backward with residual, parameter gradients and column sums."""
    T, d = 32768, 2048                              # 134 MB per bf16 tensor
    C = pccl._C
    x = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    br = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    w, b = torch.ones(d, device=DEV, dtype=torch.bfloat16), torch.zeros(d, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    gw, gb, dsum = torch.empty_like(w), torch.empty_like(b), torch.empty_like(b)
    for _ in range(3):
        y, mean, rstd = C.ln_fwd(x, br, w, b, 1e-5)
        C.ln_bwd(dy, br, mean.view(-1), rstd.view(-1), w, gw, gb, dy, dsum)
    torch.cuda.synchronize()


def gelu():
    T, f = 8192, 8192
    C = pccl._C
    u = torch.randn(T, f, device=DEV).to(torch.bfloat16)
    dg = torch.randn(T, f, device=DEV).to(torch.bfloat16)
    gb = torch.empty(f, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        C.gelu(u)
        C.gelu_bwd_col_sum(dg, u, gb)
    torch.cuda.synchronize()


def col_sum():
    T, d = 32768, 2048
    C = pccl._C
    x = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    out = torch.empty(d, device=DEV, dtype=torch.bfloat16)
    q = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    gb = torch.empty(3 * d, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        C.col_sum(x, out)
        C.cat3_col_sum(q, q, q, gb)
    torch.cuda.synchronize()


CASES = {
    "gemm": gemm, "cublas_gemm": cublas_gemm, "gemm_proj": gemm_proj, "cublas_gemm_proj": lambda: gemm_proj(True),
    "gemm_wide": gemm_wide, "gemm_nn": gemm_nn, "gemm_tn": gemm_tn, "gemm_split": gemm_split,
    "all_gather": all_gather, "all_gather_ring": lambda: _ag(sch.RING), "all_gather_recursive": lambda: _ag(sch.RECURSIVE),
    "reduce_scatter": reduce_scatter, "reduce_scatter_ring": lambda: _rs(sch.RING),
    "reduce_scatter_recursive": lambda: _rs(sch.RECURSIVE),
    "all_reduce": lambda: _ar(sch.DIRECT), "all_reduce_ring": lambda: _ar(sch.RING), "broadcast": broadcast,
    "adamw": adamw, "cross_entropy": cross_entropy, "layer_norm": layer_norm, "gelu": gelu, "col_sum": col_sum,
}

if __name__ == "__main__":
    CASES[sys.argv[1]]()
    print("done", sys.argv[1])
