"""Real multi-GPU runs: one process per GPU, peer memory mapped over NVLink, every
collective checked against NCCL on the same inputs.  Skipped on machines with one GPU."""
import os

import pytest
import torch
import torch.distributed as dist

from tests._mp import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2


def _collectives(rank, world, transport):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import pccl
    from pccl import schedule as sch

    dev = torch.device("cuda", rank)
    comm = pccl.Communicator.create(transport=transport, heap_bytes=256 << 20, staging_bytes=64 << 20,
                                    enable_nvls=False, timeout_ms=5000)
    assert comm.transport_name == transport
    g = comm.world_group
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    algos = [sch.DIRECT, sch.RING, sch.PULL] + ([sch.RECURSIVE] if sch.is_pow2(world) else [])
    for n in (1, 1000, (1 << 20) + 7):
        x = torch.randn(n, device=dev, generator=gen).to(torch.bfloat16)
        gold = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gold, x)
        big = torch.randn(world * n, device=dev, generator=gen).to(torch.bfloat16)
        allin = torch.empty(world * world * n, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(allin, big)
        want_rs = allin.view(world, world, n).float().sum(0)[rank] / world
        sym_out = comm.empty(world * n, torch.bfloat16)
        sym_big = comm.empty(world * n, torch.bfloat16)
        sym_big.copy_(big)
        for algo in algos:
            out = torch.zeros(world * n, device=dev, dtype=torch.bfloat16)
            pccl.all_gather(out, x, g, algorithm=algo)
            assert torch.equal(out, gold), f"all_gather {algo} n={n}"
            sym_out.zero_()
            pccl.all_gather(sym_out, x, g, algorithm=algo)
            assert torch.equal(sym_out, gold), f"all_gather(symmetric) {algo} n={n}"
            res = torch.zeros(n, device=dev, dtype=torch.float32)
            pccl.reduce_scatter(res, sym_big if algo == sch.PULL else big, g, algorithm=algo, scale=1.0 / world)
            tol = dict(rtol=1e-5, atol=1e-5) if algo in (sch.DIRECT, sch.PULL) else dict(rtol=3e-2, atol=3e-2)
            torch.testing.assert_close(res, want_rs, **tol)
        t = torch.randn(n, device=dev, generator=gen)
        ref = t.clone()
        dist.all_reduce(ref)
        pccl.all_reduce(t, g)
        torch.testing.assert_close(t, ref, rtol=1e-5, atol=1e-5)
        b = torch.full((n,), float(rank), device=dev)
        pccl.broadcast(b, world - 1, g)
        assert torch.all(b == float(world - 1))
        del sym_out, sym_big
    req = pccl.all_gather(torch.empty(world * 8, device=dev), torch.ones(8, device=dev), g, async_op=True)
    req.wait()
    pccl.barrier(g)
    comm.check()
    dist.barrier()
    comm.close()


@pytest.mark.parametrize("transport", ["vmm", "ipc", "symm_mem"])
def test_collectives_match_nccl(transport, port):
    run_ranks(_collectives, _world(), port, args=(transport,), backend="nccl", timeout=120)


def _zero3(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import pccl
    from pccl.models.gpt import PRESETS
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine
    from pccl.patch_deepspeed import patch_deepspeed, unpatch_deepspeed

    dev = torch.device("cuda", rank)
    cfg = PRESETS["gpt-tiny"]
    gen = torch.Generator().manual_seed(9 + rank)
    toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev)
    base = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), device=dev)
    l_base = [float(base.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(4)]
    comm = pccl.init(heap_bytes=256 << 20, staging_bytes=32 << 20, enable_nvls=False, timeout_ms=5000)
    patch_deepspeed(world)
    ours = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), device=dev, comm=comm)
    l_ours = [float(ours.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(4)]
    comm.check()
    unpatch_deepspeed()
    assert l_base[-1] < l_base[0]
    for a, b in zip(l_base, l_ours):
        assert abs(a - b) < 3e-2, (l_base, l_ours)
    # shards stayed in step.  Adam normalises gradients, so an element whose gradient is
    # nearly zero may move by +-lr in one arm and not the other: compare on average.
    diff = (base.param_shard.float() - ours.param_shard.float()).abs().mean()
    assert float(diff) < 5e-4, float(diff)
    dist.barrier()
    pccl.shutdown()


def test_zero3_training_matches_nccl_engine(port):
    run_ranks(_zero3, _world(), port, backend="nccl", timeout=120)


def _zero3_fused(rank, world):
    """The engine with the fused all-gather+GEMM on QKV and FC1 (row-sharded weights) trains
    like the NCCL-backed engine."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import pccl
    from pccl.models.gpt import GPTConfig
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine, heap_bytes_needed
    from pccl.patch_deepspeed import patch_deepspeed, unpatch_deepspeed

    dev = torch.device("cuda", rank)
    d = 256 * world                      # every rank owns whole 256-row panels of QKV and FC1
    cfg = GPTConfig(2, d, d // 64, 4 * d, vocab=1024, seq_len=128, name="gpt-fused-test")
    gen = torch.Generator().manual_seed(19 + rank)
    toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev)
    base = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), device=dev)
    l_base = [float(base.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(3)]
    del base
    comm = pccl.init(heap_bytes=heap_bytes_needed(cfg, world, True) + (128 << 20), staging_bytes=32 << 20,
                     enable_nvls=False, timeout_ms=5000)
    patch_deepspeed(world)
    ours = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), device=dev, comm=comm, fused_ag_gemm=True,
                       gather_ctas=8)
    assert ours.fused_ag_gemm and len(ours.regions[1]) == 3
    l_ours = [float(ours.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(3)]
    ours.check_errors()
    unpatch_deepspeed()
    for a, b in zip(l_base, l_ours):
        assert abs(a - b) < 3e-2, (l_base, l_ours)
    dist.barrier()
    pccl.shutdown()


def test_zero3_with_fused_all_gather_gemm(port):
    run_ranks(_zero3_fused, _world(), port, backend="nccl", timeout=120)


def _leaver(rank, world):
    """A rank leaves between steps; the others learn of it from their bounded waits (a
    short timeout), get an exception, and their CUDA context keeps working."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import pccl

    dev = torch.device("cuda", rank)
    comm = pccl.Communicator.create(heap_bytes=64 << 20, staging_bytes=16 << 20, enable_nvls=False, timeout_ms=300)
    g = comm.world_group
    out = torch.zeros(world * 16, device=dev)
    pccl.all_gather(out, torch.full((16,), float(rank), device=dev), g)       # step 1: everybody is here
    comm.check()
    dist.barrier()
    if rank == world - 1:
        torch.cuda.synchronize()
        return                                                                 # leaves with nothing in flight
    pccl.all_gather(out, torch.ones(16, device=dev), g)                        # step 2: one peer is missing
    with pytest.raises(pccl.PcclTimeoutError):
        comm.check()
    assert float(torch.ones(8, device=dev).sum()) == 8.0                       # the context survived


def test_rank_leaving_is_detected_by_bounded_waits(port):
    run_ranks(_leaver, 2, port, backend="nccl", timeout=120)
