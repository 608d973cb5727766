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
    # eager: the handshake-free variant for small messages (larger ones fall back to direct)
    algos = [sch.DIRECT, sch.RING, sch.PULL, sch.EAGER] + ([sch.RECURSIVE] if sch.is_pow2(world) else [])
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
            tol = dict(rtol=1e-5, atol=1e-5) if algo in (sch.DIRECT, sch.PULL, sch.EAGER) else dict(rtol=3e-2, atol=3e-2)
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


def _multimem(rank, world):
    """NVLS variants on healthy ranks: multimem.st all-gather and broadcast, multimem.ld_reduce
    reduce-scatter and all-reduce, against NCCL.  Every rank stays to the end and unbinds its
    memory in comm.close() before it exits."""
    import pccl
    from pccl import schedule as sch

    dev = torch.device("cuda", rank)
    comm = pccl.Communicator.create(transport="vmm", heap_bytes=256 << 20, staging_bytes=32 << 20, enable_nvls=True,
                                    timeout_ms=5000)
    if not comm.nvls:
        dist.barrier()
        comm.close()
        return "multicast is not offered on this machine"
    g = comm.world_group
    gen = torch.Generator(device=dev).manual_seed(300 + rank)
    for n in (8, 4096, (1 << 20) + 8):                      # multiples of 8 elements: 16-byte blocks
        x = torch.randn(n, device=dev, generator=gen).to(torch.bfloat16)
        gold = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gold, x)
        sym_out = comm.empty(world * n, torch.bfloat16)
        sym_out.zero_()
        pccl.all_gather(sym_out, x, g, algorithm=sch.MULTIMEM)
        assert torch.equal(sym_out, gold), f"multimem all_gather n={n}"
        sym_in = comm.empty(world * n, torch.bfloat16)
        big = torch.randn(world * n, device=dev, generator=gen).to(torch.bfloat16)
        sym_in.copy_(big)
        allin = torch.empty(world * world * n, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(allin, big)
        want = allin.view(world, world, n).float().sum(0)[rank] / world
        for tout in (torch.float32, torch.bfloat16):
            res = torch.zeros(n, device=dev, dtype=tout)
            pccl.reduce_scatter(res, sym_in, g, algorithm=sch.MULTIMEM, scale=1.0 / world)
            # the switch adds in fp32 but hands the sum back in the input type: one bf16 rounding either way
            torch.testing.assert_close(res.float(), want, rtol=1e-2, atol=1e-2, msg=lambda m: f"multimem reduce_scatter n={n} {tout}: {m}")
        ar = comm.empty(world * n, torch.float32)
        t = torch.randn(world * n, device=dev, generator=gen)
        ar.copy_(t)
        ref = t.clone()
        dist.all_reduce(ref)
        pccl.all_reduce(ar, g, algorithm=sch.MULTIMEM)
        torch.testing.assert_close(ar, ref, rtol=1e-5, atol=1e-4, msg=lambda m: f"multimem all_reduce n={n}: {m}")
        b = comm.empty(n, torch.float32)
        b.fill_(float(rank))
        pccl.broadcast(b, 1 % world, g)
        assert torch.all(b == float(1 % world)), f"multimem broadcast n={n}"
        del sym_out, sym_in, ar, b
    comm.check()
    dist.barrier()
    comm.close()


def test_multimem_variants_match_nccl(port):
    run_ranks(_multimem, _world(), port, backend="nccl", timeout=180)


def _reference_named_entry_points(rank, world):
    """pccl._C.all_gather_mpi / reduce_scatter_mpi / all_reduce_mpi(…, group, "recursive" | "ring"):
    the native entry points under the reference's names, and the all-reduce that runs the
    reference's composition (reduce-scatter + all-gather of one schedule family) as one launch."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import pccl

    C = pccl._C
    dev = torch.device("cuda", rank)
    comm = pccl.Communicator.create(heap_bytes=128 << 20, staging_bytes=32 << 20, enable_nvls=False, timeout_ms=5000)
    g = comm.world_group
    gen = torch.Generator(device=dev).manual_seed(500 + rank)
    algos = ["ring"] + (["recursive"] if world & (world - 1) == 0 else [])
    for n in (8, 1000, (1 << 19) + 8):
        x = torch.randn(n, device=dev, generator=gen)
        gold = torch.empty(world * n, device=dev)
        dist.all_gather_into_tensor(gold, x)
        big = torch.randn(world * n, device=dev, generator=gen)
        want_rs = torch.empty(n, device=dev)
        dist.reduce_scatter_tensor(want_rs, big)
        for algo in algos:
            out = torch.zeros(world * n, device=dev)
            C.all_gather_mpi(out, x, g, algo)
            assert torch.equal(out, gold), f"all_gather_mpi {algo}"
            res = torch.zeros(n, device=dev)
            C.reduce_scatter_mpi(res, big, g, algo)
            torch.testing.assert_close(res, want_rs, rtol=1e-5, atol=1e-4)
            t = big.clone()
            ref = big.clone()
            dist.all_reduce(ref)
            C.all_reduce_mpi(t, g, algo)
            torch.testing.assert_close(t, ref, rtol=1e-5, atol=1e-4)
            sym = comm.empty(world * n, torch.bfloat16)
            sym.copy_(big.to(torch.bfloat16))
            pccl.all_reduce(sym, g, algorithm=algo)                 # symmetric tensor: zero-copy gather phase
            torch.testing.assert_close(sym.float(), ref, rtol=4e-2, atol=4e-2 * float(ref.abs().max()))
            del sym
    with pytest.raises(RuntimeError, match="Unknown algorithm"):
        C.all_gather_mpi(torch.zeros(world * 4, device=dev), torch.zeros(4, device=dev), g, "tree")
    with pytest.raises(RuntimeError, match="1D"):
        C.reduce_scatter_mpi(torch.zeros(4, 1, device=dev), torch.zeros(4 * world, 1, device=dev), g, "ring")
    with pytest.raises(RuntimeError, match="divisible"):
        C.reduce_scatter_mpi(torch.zeros(4, device=dev), torch.zeros(4 * world + 1, device=dev), g, "ring")
    comm.check()
    dist.barrier()
    comm.close()


def test_entry_points_under_the_reference_names(port):
    run_ranks(_reference_named_entry_points, _world(), port, backend="nccl", timeout=180)


def _copy_engine_paths(rank, world):
    """Parameter gathers by the copy engines: the all-gather without a kernel, the fused
    all-gather+GEMM fed by copies and stream-ordered flag writes, and the ZeRO-3 engine on both
    with every dense product on the library GEMM, against the NCCL + cuBLAS engine."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import pccl
    from pccl import schedule as sch
    from pccl.models.gpt import GPTConfig
    from pccl.ops.ag_gemm import AllGatherLinear
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine, heap_bytes_needed
    from pccl.patch_deepspeed import patch_deepspeed, unpatch_deepspeed

    dev = torch.device("cuda", rank)
    d = 256 * world
    cfg = GPTConfig(2, d, d // 64, 4 * d, vocab=1024, seq_len=128, name="gpt-copy-engine-test")
    gen = torch.Generator().manual_seed(29 + rank)
    toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev)
    base = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), device=dev, native_gemm=False)
    l_base = [float(base.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(3)]
    del base
    comm = pccl.init(heap_bytes=heap_bytes_needed(cfg, world, True) + (256 << 20), staging_bytes=32 << 20,
                     enable_nvls=False, timeout_ms=5000)
    g = comm.world_group
    # all-gather without a kernel
    n = (1 << 18) + 8
    x = comm.empty(n, torch.bfloat16)
    x.copy_(torch.randn(n, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16))
    gold = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(gold, x)
    out = torch.zeros(world * n, device=dev, dtype=torch.bfloat16)
    pccl.barrier(g)                                         # every rank's input is complete
    req = pccl.all_gather(out, x, g, async_op=True, algorithm=sch.COPY_ENGINE)
    req.wait()
    torch.cuda.synchronize()
    assert torch.equal(out, gold)
    # fused all-gather+GEMM fed by the copy engines
    N, K, M = 256 * world * 2, 512, 640
    lin = AllGatherLinear(comm, None, N, K, copy_engine=True)
    lin.w_shard.copy_((torch.randn(N // world, K, generator=torch.Generator().manual_seed(50 + rank)) * 0.05).to(torch.bfloat16))
    torch.cuda.synchronize()
    dist.barrier()
    A = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w_gold = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(w_gold, lin.w_shard)
    for _ in range(2):
        y = lin(A, check=True)
        torch.cuda.synchronize()
        assert torch.equal(lin.w_full, w_gold)
        ref = A.float() @ w_gold.float().t()
        assert float((y.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max()) + 1e-3
    dist.barrier()
    del lin
    # the engine: copy-engine gathers, library GEMMs; then with the fused kernel on QKV / FC1 too
    patch_deepspeed(world)
    for fused in (False, True):
        ours = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), device=dev, comm=comm, native_gemm=True,
                           copy_engine_gather=True, fused_ag_gemm=fused)
        assert ours.copy_engine_gather and ours.native_gemm and ours.fused_ag_gemm == fused
        l_ours = [float(ours.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(3)]
        ours.check_errors()
        for a, b in zip(l_base, l_ours):
            assert abs(a - b) < 3e-2, (fused, l_base, l_ours)
        del ours
    unpatch_deepspeed()
    dist.barrier()
    pccl.shutdown()


def test_copy_engine_gathers_and_native_gemm_engine(port):
    run_ranks(_copy_engine_paths, _world(), port, backend="nccl", timeout=240)
