"""World-size-2..4 collectives on CPU over gloo, checked against torch.distributed.

Covers the first benchmark configuration: 1,048,576 fp32 elements per rank drawn N(0,1)
from seed+rank, ring and recursive algorithms, compared with the torch.distributed result.
"""
import pytest
import torch
import torch.distributed as dist

from tests._mp import run_ranks


def _config1(rank, world, n):
    import pccl

    comm = pccl.init()
    g = comm.world_group
    assert not g.native
    gen = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(n, generator=gen, dtype=torch.float32)
    for algo in ("ring", "recursive", "direct"):
        out = torch.empty(world * n)
        gold = torch.empty(world * n)
        pccl._all_gather(out, x, g, use_rd=(algo == "recursive"), algorithm=None if algo != "direct" else "direct")
        pccl._all_gather(gold, x, None)
        assert torch.equal(out, gold), f"all_gather {algo} differs from torch.distributed"

        big = torch.randn(world * n, generator=gen, dtype=torch.float32)
        out = torch.empty(n)
        gold = torch.empty(n)
        pccl._reduce_scatter(out, big, g, use_rh=(algo == "recursive"), algorithm=None if algo != "direct" else "direct")
        pccl._reduce_scatter(gold, big, None)
        if world == 2:
            assert torch.equal(out, gold)          # one addition: exact
        else:
            torch.testing.assert_close(out, gold, rtol=1e-5, atol=1e-6)

        t = torch.randn(n + 3, generator=gen)
        ref = t.clone()
        pccl._all_reduce(t, g, use_rh_and_rd=(algo == "recursive"))
        dist.all_reduce(ref)
        torch.testing.assert_close(t, ref, rtol=1e-5, atol=1e-6)
    # exported reference names
    out = torch.empty(world * n)
    pccl.recursive_doubling_allgather_mpi(out, x, g)
    gold = torch.empty(world * n)
    dist.all_gather_into_tensor(gold, x)
    assert torch.equal(out, gold)
    big = torch.randn(world * n, generator=gen)
    o1, o2, gold = torch.empty(n), torch.empty(n), torch.empty(n)
    pccl.recursive_halving_reduce_scatter_mpi(o1, big, g)
    pccl.ring_reduce_scatter_mpi(o2, big, g)
    dist.reduce_scatter_tensor(gold, big)
    torch.testing.assert_close(o1, gold, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(o2, gold, rtol=1e-5, atol=1e-6)


def test_config1_world2_one_mebi_elements(port):
    run_ranks(_config1, 2, port, args=(1 << 20,))


def test_world4_small(port):
    run_ranks(_config1, 4, port, args=(1000,))


def _bf16_and_scale(rank, world):
    import pccl

    g = pccl.init().world_group
    gen = torch.Generator().manual_seed(7 + rank)
    n = 515
    big = torch.randn(world * n, generator=gen).to(torch.bfloat16)
    allin = [torch.empty_like(big) for _ in range(world)]
    dist.all_gather(allin, big)
    want = sum(t.float() for t in allin).view(world, n)[rank] / world
    for algo in ("ring", "direct"):
        out = torch.empty(n, dtype=torch.float32)
        pccl._reduce_scatter(out, big, g, algorithm=algo, scale=1.0 / world, wire_dtype=torch.float32)
        torch.testing.assert_close(out, want, rtol=1e-6, atol=1e-6)   # fp32 wire: only reassociation
        out16 = torch.empty(n, dtype=torch.bfloat16)
        pccl._reduce_scatter(out16, big, g, algorithm=algo, scale=1.0 / world)
        torch.testing.assert_close(out16.float(), want, rtol=2e-2, atol=2e-2)
    t = torch.full((10,), float(rank + 1))
    pccl.broadcast(t, 1, g)
    assert torch.equal(t, torch.full((10,), 2.0))
    pccl.barrier(g)
    req = pccl._all_gather(torch.empty(world * 4), torch.ones(4), g, async_op=True)
    assert isinstance(req, pccl.Request)
    seen = []
    req.wait(lambda: seen.append(1))
    assert seen == [1]


def test_bf16_scale_broadcast_barrier_world3(port):
    run_ranks(_bf16_and_scale, 3, port)


def _two_d(rank, world):
    import pccl

    pgs = pccl.ProcessGroups(2, 2)
    assert pgs.get_world_size() == [2, 2]
    assert pgs.get_rank() == [rank % 2, (rank // 2) % 2]
    assert pgs.get_rank(0) == rank % 2 and pgs.get_world_size(1) == 2
    with pytest.raises(ValueError):
        pgs.get_rank(2)
    assert pgs.get_inner_group().ranks == [rank - rank % 2, rank - rank % 2 + 1]
    assert pgs.get_outer_group().ranks == [rank % 2, rank % 2 + 2]
    n = 37
    x = torch.arange(n, dtype=torch.float32) + 100 * rank
    out = torch.empty(world * n)
    pccl.all_gather_2D(out, x, pgs, use_rd=True)
    gold = torch.empty(world * n)
    dist.all_gather_into_tensor(gold, x)
    assert torch.equal(out, gold)
    big = torch.randn(world * n, generator=torch.Generator().manual_seed(rank))
    o = torch.empty(n)
    pccl.reduce_scatter_2D(o, big, pgs, use_rh=True)
    gold = torch.empty(n)
    dist.reduce_scatter_tensor(gold, big)
    torch.testing.assert_close(o, gold, rtol=1e-5, atol=1e-6)
    # mixed backends: torch groups inside, library groups outside
    mixed = pccl.ProcessGroups(2, 2, inner_group_backend="gloo", outer_group_backend="pccl")
    out2 = torch.empty(world * n)
    pccl.all_gather_2D(out2, x, mixed, use_rd=True)
    assert torch.equal(out2, gold.new_tensor(out))
    with pytest.raises(ValueError):
        pccl.ProcessGroups(3, 1)
    with pytest.raises(ValueError):
        pccl.ProcessGroups(2, 2, inner_group_backend="smoke-signals")
    # two independent grids of 2 ranks
    pair = pccl.ProcessGroups(2, 1)
    assert pair.num_2d_grids == 2
    o = torch.empty(2 * n)
    pccl.all_gather_2D(o, x, pair)
    base = rank - rank % 2
    assert torch.equal(o[:n], torch.arange(n, dtype=torch.float32) + 100 * base)


def test_process_groups_and_2d_world4(port):
    run_ranks(_two_d, 4, port)


def _dead_peer(rank, world):
    """A rank that never joins a step must surface as PcclTimeoutError on its peer."""
    import os

    os.environ["PCCL_P2P_TIMEOUT_S"] = "2"
    import pccl

    g = pccl.init().world_group
    if rank == 1:
        return                      # leaves between steps: never posts its send/recv
    out = torch.empty(world * 8)
    with pytest.raises(pccl.PcclTimeoutError):
        pccl._all_gather(out, torch.ones(8), g)


def test_missing_rank_times_out(port):
    run_ranks(_dead_peer, 2, port)


def _patched_backend(rank, world):
    """patch_deepspeed on CPU ranks: the five backend methods go through the 2-D library path for
    world-sized groups and SUM, and fall back to the saved originals otherwise."""
    import pccl  # noqa: F401
    from pccl import patch_deepspeed as pd
    from pccl.parallel.backend import TorchBackend

    be = TorchBackend()
    pgs = pd.patch_deepspeed(2, algorithm=None)            # 2 x 2 grid; reference choice: recursive variants
    assert pd.get_heir_pg() is pgs and pgs.get_world_size() == [2, 2]
    for name in ("all_gather_into_tensor", "reduce_scatter_tensor", "all_reduce", "broadcast", "barrier"):
        assert hasattr(TorchBackend, "old_" + name)
    assert TorchBackend.fused_scale and TorchBackend.symmetric_memory
    assert pd.is_global_pg(None) and pd.is_global_pg(dist.group.WORLD)
    gen = torch.Generator().manual_seed(99 + rank)
    n = 1000
    x = torch.randn(n, generator=gen)
    out, gold = torch.empty(world * n), torch.empty(world * n)
    assert be.all_gather_into_tensor(out, x) is None       # global-rank order although the grid is 2-D
    be.old_all_gather_into_tensor(gold, x)
    assert torch.equal(out, gold)
    big = torch.randn(world * n, generator=gen)
    out, gold = torch.empty(n), torch.empty(n)
    be.reduce_scatter_tensor(out, big, scale=0.25)
    be.old_reduce_scatter_tensor(gold, big)
    torch.testing.assert_close(out, gold * 0.25, rtol=1e-5, atol=1e-6)
    t = torch.randn(n + 1, generator=gen)
    ref = t.clone()
    be.all_reduce(t)
    be.old_all_reduce(ref)
    torch.testing.assert_close(t, ref, rtol=1e-5, atol=1e-6)
    b = torch.full((5,), float(rank))
    be.broadcast(b, 3)
    assert torch.equal(b, torch.full((5,), 3.0))
    be.barrier()
    # not the whole world, or not a sum: the original methods run
    sub = dist.new_group([0, 1])
    if rank < 2:
        o2 = torch.empty(2 * n)
        be.all_gather_into_tensor(o2, x, group=sub)
        g2 = torch.empty(2 * n)
        dist.all_gather_into_tensor(g2, x, group=sub)
        assert torch.equal(o2, g2)
    m = torch.full((3,), float(rank))
    be.all_reduce(m, op=dist.ReduceOp.MAX)
    assert torch.equal(m, torch.full((3,), float(world - 1)))
    req = be.all_gather_into_tensor(out := torch.empty(world * n), x, async_op=True)
    req.wait()
    be.old_all_gather_into_tensor(gold := torch.empty(world * n), x)
    assert torch.equal(out, gold)
    pd.unpatch_deepspeed()
    assert not hasattr(TorchBackend, "old_all_reduce") and not TorchBackend.fused_scale


def test_patched_backend_world4_on_cpu(port):
    run_ranks(_patched_backend, 4, port)


def _fd_channel_and_max(rank, world):
    """The bootstrap's descriptor channel (unix datagram sockets, SCM_RIGHTS) with ordinary
    files standing in for exported GPU allocations, and the max-over-ranks reduction."""
    import os
    import tempfile

    from pccl.comm import _FdChannel
    from pccl.utils.timing import max_over_ranks

    job = f"test{os.environ['MASTER_PORT']}"
    ch = _FdChannel(job, rank, world, timeout_s=20.0)
    dist.barrier()                                         # every socket is bound before anyone sends
    with tempfile.TemporaryFile() as f:
        f.write(f"heap of rank {rank}".encode())
        f.flush()
        for dst in range(world):
            if dst != rank:
                ch.send(dst, [os.dup(f.fileno())], tag=7)  # send() closes the descriptors it was given
        got = {}
        for _ in range(world - 1):
            src, tag, fds = ch.recv()
            assert tag == 7 and len(fds) == 1
            # positional read: the received descriptor shares its file offset with the sender's
            got[src] = os.pread(fds[0], 100, 0).decode()
            os.close(fds[0])
    assert got == {r: f"heap of rank {r}" for r in range(world) if r != rank}
    ch.close()
    assert max_over_ranks(10.0 + rank) == 10.0 + world - 1


def test_descriptor_channel_and_max_over_ranks(port):
    run_ranks(_fd_channel_and_max, 3, port)


def _peer_missing_at_handle_exchange(rank, world):
    """Rendezvous failure injected on the host: the last rank never sends its memory handles.
    The others' receive runs into the channel's timeout, and the phase's agreement step turns that
    into the same PcclError on EVERY rank (the silent one included), so nobody falls out of step
    or hangs; the ranks can then go on (here: one more collective on the process group)."""
    import os
    import tempfile
    import types

    from pccl.comm import Communicator, PcclError, _FdChannel

    job = f"miss{os.environ['MASTER_PORT']}"
    ch = _FdChannel(job, rank, world, timeout_s=0.5)
    dist.barrier()
    me = types.SimpleNamespace(world=world, pg=None)
    me._all_gather_obj = types.MethodType(Communicator._all_gather_obj, me)

    def exchange():
        with tempfile.TemporaryFile() as f:
            if rank != world - 1:                           # the faulty rank keeps its handles to itself
                for dst in range(world):
                    if dst != rank:
                        ch.send(dst, [os.dup(f.fileno())], tag=0)
            for _ in range(world - 1):
                _src, _tag, fds = ch.recv()
                for fd in fds:
                    os.close(fd)

    with pytest.raises(PcclError) as err:
        Communicator._agree(me, exchange)
    assert "timed out" in str(err.value).lower() or "timeout" in str(err.value).lower()
    ch.close()
    t = torch.ones(1)
    dist.all_reduce(t)                                      # the process group is still usable
    assert int(t.item()) == world


def test_peer_missing_at_handle_exchange_raises_everywhere(port):
    run_ranks(_peer_missing_at_handle_exchange, 3, port)
