"""Collective kernels on ONE GPU: all P ranks are emulated by a single cooperative launch
(blockIdx.y = rank) over P separate heaps, so the full flag protocol, every schedule and
every dtype path runs exactly as it does across GPUs.  References are plain PyTorch fp32."""
import pytest
import torch

import pccl
from pccl import schedule as sch
from pccl.all_gather import ag2d_inner_call, ag2d_outer_call
from pccl.reduce_scatter import rs2d_inner_call, rs2d_outer_call

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
_comms = {}


def emu(P):
    if P not in _comms:
        _comms[P] = pccl.Communicator.emulated_world(P, device=0, heap_bytes=96 << 20, staging_bytes=24 << 20)
    return _comms[P]


def rand(n, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(n, generator=g, device=DEV, dtype=torch.float32).to(dtype)


SIZES = [1, 3, 17, 4096, (1 << 18) + 5]


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("algo", [sch.DIRECT, sch.RING, sch.RECURSIVE, sch.PULL])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_all_gather_private_buffers(P, algo, dtype):
    comm = emu(P)
    for n in SIZES:
        ins = [rand(n, dtype, 10 * r + n) for r in range(P)]
        outs = [torch.zeros(P * n, dtype=dtype, device=DEV) for _ in range(P)]
        comm.native.all_gather(comm.world_group.gid, outs, ins, sch.ALGO_IDS[algo], 5)
        comm.check()
        want = torch.cat(ins)
        for r in range(P):
            assert torch.equal(outs[r], want), f"P={P} {algo} n={n} rank {r}"


@pytest.mark.parametrize("P", [2, 8])
@pytest.mark.parametrize("algo", [sch.DIRECT, sch.RING, sch.RECURSIVE, sch.PULL])
def test_all_gather_symmetric_zero_copy(P, algo):
    comm = emu(P)
    n = 70001
    outs = comm.empty(P * n, torch.bfloat16)
    sym_in = comm.empty(n, torch.bfloat16)
    vals = [rand(n, torch.bfloat16, 3 + r) for r in range(P)]
    for r in range(P):
        outs[r].zero_()
        sym_in[r].copy_(vals[r])
    comm.native.all_gather(comm.world_group.gid, outs, sym_in, sch.ALGO_IDS[algo], 7)
    comm.check()
    want = torch.cat(vals)
    for r in range(P):
        assert torch.equal(outs[r], want)
    # in place: the contribution already sits in its slot of the output
    for r in range(P):
        outs[r].zero_()
        outs[r][r * n:(r + 1) * n].copy_(vals[r])
    if algo != sch.PULL:
        comm.native.all_gather(comm.world_group.gid, outs, [outs[r][r * n:(r + 1) * n] for r in range(P)],
                               sch.ALGO_IDS[algo], 3)
        comm.check()
        for r in range(P):
            assert torch.equal(outs[r], want)
    del outs, sym_in


def rs_reference(ins, P, n, scale, out_dtype):
    total = sum(t.float() for t in ins).view(P, n) * scale
    return [total[r].to(out_dtype) for r in range(P)]


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("algo", [sch.DIRECT, sch.RING, sch.RECURSIVE])
@pytest.mark.parametrize("dtypes", [(torch.bfloat16, None, torch.bfloat16), (torch.bfloat16, torch.float32, torch.float32),
                                    (torch.float32, None, torch.float32), (torch.float16, None, torch.float32)])
def test_reduce_scatter_push(P, algo, dtypes):
    tin, wire, tout = dtypes
    comm = emu(P)
    for n in SIZES:
        ins = [rand(P * n, tin, 100 * r + n) for r in range(P)]
        outs = [torch.zeros(n, dtype=tout, device=DEV) for _ in range(P)]
        scale = 1.0 / P
        comm.native.reduce_scatter(comm.world_group.gid, outs, ins, sch.ALGO_IDS[algo], 4, scale, wire)
        comm.check()
        want = rs_reference(ins, P, n, scale, tout)
        exact_partials = wire == torch.float32 or tin == torch.float32 or algo == sch.DIRECT
        for r in range(P):
            if exact_partials:
                # single rounding: only fp32 reassociation separates us from the reference
                tol = dict(rtol=1e-5, atol=1e-5) if tout == torch.float32 else dict(rtol=8e-3, atol=1e-5)
            else:
                tol = dict(rtol=3e-2, atol=3e-2)       # partial sums were rounded to 16 bits on the wire
            torch.testing.assert_close(outs[r].float(), want[r].float(), **tol)


@pytest.mark.parametrize("P", [2, 8])
def test_reduce_scatter_pull_symmetric_input(P):
    comm = emu(P)
    n = 40003
    sym = comm.empty(P * n, torch.bfloat16)
    vals = [rand(P * n, torch.bfloat16, 50 + r) for r in range(P)]
    for r in range(P):
        sym[r].copy_(vals[r])
    outs = [torch.zeros(n, dtype=torch.float32, device=DEV) for _ in range(P)]
    comm.native.reduce_scatter(comm.world_group.gid, outs, sym, sch.ALGO_IDS[sch.PULL], 6, 0.5, None)
    comm.check()
    want = rs_reference(vals, P, n, 0.5, torch.float32)
    for r in range(P):
        torch.testing.assert_close(outs[r], want[r], rtol=1e-5, atol=1e-5)
    priv = [v.clone() for v in vals]
    with pytest.raises(RuntimeError):
        comm.native.reduce_scatter(comm.world_group.gid, outs, priv, sch.ALGO_IDS[sch.PULL], 6, 1.0, None)
    del sym


def test_reduce_scatter_bf16_accumulates_in_fp32():
    """Many equal small addends: a 16-bit accumulator would stall, fp32 does not."""
    P = 8
    comm = emu(P)
    n = 1024
    ins = []
    for r in range(P):
        t = torch.full((P * n,), 1.0 if r == 0 else 2.0 ** -9, dtype=torch.bfloat16, device=DEV)
        ins.append(t)
    outs = [torch.zeros(n, dtype=torch.float32, device=DEV) for _ in range(P)]
    comm.native.reduce_scatter(comm.world_group.gid, outs, ins, sch.ALGO_IDS[sch.DIRECT], 2, 1.0, None)
    comm.check()
    assert torch.all(outs[3] == 1.0 + 7 * 2.0 ** -9)


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_all_reduce(P, dtype):
    comm = emu(P)
    for n in [1, 9, 1000, (1 << 17) + 3]:
        ts = [rand(n, dtype, 7 * r + n) for r in range(P)]
        want = sum(t.float() for t in ts)
        comm.native.all_reduce(comm.world_group.gid, ts, sch.ALGO_IDS[sch.DIRECT], 4, 1.0)
        comm.check()
        for r in range(P):
            tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=8e-3, atol=1e-3)
            torch.testing.assert_close(ts[r].float(), want, **tol)
            assert torch.equal(ts[r], ts[0]), "all ranks must hold bit-identical results"
    sym = comm.empty(5000, dtype)
    vals = [rand(5000, dtype, 99 + r) for r in range(P)]
    for r in range(P):
        sym[r].copy_(vals[r])
    comm.native.all_reduce(comm.world_group.gid, sym, sch.ALGO_IDS[sch.DIRECT], 3, 1.0 / P)
    comm.check()
    want = sum(v.float() for v in vals) / P
    for r in range(P):
        torch.testing.assert_close(sym[r].float(), want, rtol=8e-3, atol=1e-3)
    del sym


@pytest.mark.parametrize("P", [2, 8])
def test_broadcast_and_barrier(P):
    comm = emu(P)
    for root in (0, P - 1):
        for n in (5, 100003):
            ts = [torch.full((n,), float(r), device=DEV) for r in range(P)]
            comm.native.broadcast(comm.world_group.gid, ts, root, 4, False)
            comm.check()
            for r in range(P):
                assert torch.all(ts[r] == float(root))
    for _ in range(3):
        comm.native.barrier(comm.world_group.gid)
    comm.check()


def test_subgroups_and_2d_hierarchy():
    """Inner/outer groups of a 2x2 grid, driven group by group, give the flat result
    without any permute pass."""
    comm = emu(4)
    pgs = pccl.ProcessGroups(2, 2, comm=comm)
    intra = inter = 2
    n = 3001
    native = comm.native
    vals = [rand(n, torch.bfloat16, 11 + r) for r in range(4)]
    outs = [torch.zeros(4 * n, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    nb = n * 2
    recv_off = native.staging_off
    for col, g in enumerate(pgs.all_outer_groups):          # ranks {col, col+2}
        ag2d_outer_call(native, g.gid, sch.ALGO_IDS[sch.RECURSIVE], 3, [vals[r].data_ptr() for r in g.ranks], recv_off,
                        col, nb, intra)
    for g in pgs.all_inner_groups:
        ag2d_inner_call(native, g.gid, sch.ALGO_IDS[sch.RING], 3, [outs[r].data_ptr() for r in g.ranks], recv_off, nb,
                        intra, inter)
    comm.check()
    want = torch.cat(vals)
    for r in range(4):
        assert torch.equal(outs[r], want)

    ins = [rand(4 * n, torch.float32, 21 + r) for r in range(4)]
    mids = [torch.zeros(inter * n, device=DEV) for _ in range(4)]
    res = [torch.zeros(n, device=DEV) for _ in range(4)]
    for g in pgs.all_inner_groups:
        rs2d_inner_call(native, g.gid, sch.ALGO_IDS[sch.RECURSIVE], 3, 2, [ins[r].data_ptr() for r in g.ranks],
                        [mids[r].data_ptr() for r in g.ranks], n, 4, intra, inter)
    for g in pgs.all_outer_groups:
        rs2d_outer_call(native, g.gid, sch.ALGO_IDS[sch.RING], 3, 2, 2, [mids[r].data_ptr() for r in g.ranks],
                        [res[r].data_ptr() for r in g.ranks], n, 4, 4, 0.25)
    comm.check()
    want = rs_reference(ins, 4, n, 0.25, torch.float32)
    for r in range(4):
        torch.testing.assert_close(res[r], want[r], rtol=1e-5, atol=1e-5)


def test_chunking_when_staging_is_small():
    comm = pccl.Communicator.emulated_world(4, device=0, heap_bytes=8 << 20, staging_bytes=1 << 20)
    n = 400000                                            # 4 * 1.6 MB > 1 MiB of staging
    ins = [rand(n, torch.float32, r) for r in range(4)]
    outs = [torch.zeros(4 * n, device=DEV) for _ in range(4)]
    comm.native.all_gather(comm.world_group.gid, outs, ins, sch.ALGO_IDS[sch.RING], 4)
    big = [rand(4 * n, torch.float32, 9 + r) for r in range(4)]
    red = [torch.zeros(n, device=DEV) for _ in range(4)]
    comm.native.reduce_scatter(comm.world_group.gid, red, big, sch.ALGO_IDS[sch.DIRECT], 4, 1.0, None)
    ar = [rand(3 * n, torch.float32, 30 + r) for r in range(4)]
    want_ar = sum(ar)
    comm.native.all_reduce(comm.world_group.gid, ar, sch.ALGO_IDS[sch.DIRECT], 4, 1.0)
    comm.check()
    for r in range(4):
        assert torch.equal(outs[r], torch.cat(ins))
        torch.testing.assert_close(red[r], rs_reference(big, 4, n, 1.0, torch.float32)[r], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(ar[r], want_ar, rtol=1e-5, atol=1e-5)


def test_argument_checks():
    comm = emu(2)
    gid = comm.world_group.gid
    a = [torch.zeros(10, device=DEV) for _ in range(2)]
    with pytest.raises(RuntimeError):       # wrong output size
        comm.native.all_gather(gid, a, a, 0, 1)
    with pytest.raises(RuntimeError):       # not divisible by world size
        comm.native.reduce_scatter(gid, [torch.zeros(5, device=DEV)] * 2, [torch.zeros(11, device=DEV)] * 2, 0, 1, 1.0, None)
    with pytest.raises(RuntimeError):       # non-contiguous
        nc = [torch.zeros(20, device=DEV)[::2] for _ in range(2)]
        comm.native.all_gather(gid, [torch.zeros(20, device=DEV)] * 2, nc, 0, 1)
    with pytest.raises(RuntimeError):       # integer dtype cannot be reduced
        comm.native.all_reduce(gid, [torch.zeros(4, dtype=torch.int32, device=DEV)] * 2, 0, 1, 1.0)
    c3 = pccl.Communicator.emulated_world(3, device=0, heap_bytes=4 << 20, staging_bytes=1 << 20)
    t = [torch.zeros(3, device=DEV) for _ in range(3)]
    o = [torch.zeros(9, device=DEV) for _ in range(3)]
    with pytest.raises(RuntimeError):       # recursive doubling needs a power of two
        c3.native.all_gather(c3.world_group.gid, o, t, sch.ALGO_IDS[sch.RECURSIVE], 1)
    c3.native.all_gather(c3.world_group.gid, o, t, sch.ALGO_IDS[sch.RING], 1)   # ring takes any size
    c3.check()


def test_bounded_wait_reports_timeout_and_context_survives():
    """A rank whose peers never show up: the kernel gives up after its time limit, says where,
    and returns.  Nothing traps; the device stays usable; recover() clears the failure."""
    comm = pccl.Communicator.with_fake_peers(2, rank=0, device=0, timeout_ms=50.0)
    x = torch.ones(1000, device=DEV)
    out = torch.zeros(2000, device=DEV)
    pccl._all_gather(out, x, comm.world_group, use_pccl_cpp_backend=True, algorithm=sch.DIRECT)
    with pytest.raises(pccl.PcclTimeoutError) as err:
        comm.check()
    assert "entry" in str(err.value) and "rank 1" in str(err.value)
    # the context is healthy: ordinary work still runs
    assert float((torch.ones(10, device=DEV) * 2).sum()) == 20.0
    comm.recover()
    comm.check()
    # after a failure and recovery the same thing happens again, cleanly
    comm.native.barrier(comm.world_group.gid)
    with pytest.raises(pccl.PcclTimeoutError):
        comm.check()
    comm.recover()


@pytest.mark.parametrize("P", [4, 8])
def test_stress_mode_keeps_results_and_trace_records_the_protocol(P):
    """Every lane sleeps a pseudo-random time before each wait and signal, so ranks and lanes
    meet in orders a quiet GPU never produces: results must stay bit-exact (all-gather) or equal
    to the fp32 reference (reduce-scatter).  The device-side trace of the same calls shows every
    rank signalling and waiting."""
    comm = pccl.Communicator.emulated_world(P, device=0, heap_bytes=64 << 20, staging_bytes=16 << 20)
    comm.set_debug(jitter_us=150.0, trace_events=1 << 16)
    gid = comm.world_group.gid
    n = 40000 + 3
    for rep in range(3):                               # back-to-back calls reuse flags and staging
        for algo in (sch.DIRECT, sch.RING, sch.RECURSIVE, sch.PULL):
            ins = [rand(n, torch.bfloat16, 100 * rep + 7 * r) for r in range(P)]
            outs = [torch.zeros(P * n, dtype=torch.bfloat16, device=DEV) for _ in range(P)]
            comm.native.all_gather(gid, outs, ins, sch.ALGO_IDS[algo], 4)
            want = torch.cat(ins)
            comm.check()
            for r in range(P):
                assert torch.equal(outs[r], want), f"all_gather {algo} rep {rep} rank {r}"
        for algo in (sch.DIRECT, sch.RING, sch.RECURSIVE):
            ins = [rand(P * n, torch.bfloat16, 1000 * rep + 11 * r) for r in range(P)]
            outs = [torch.zeros(n, dtype=torch.float32, device=DEV) for _ in range(P)]
            comm.native.reduce_scatter(gid, outs, ins, sch.ALGO_IDS[algo], 4, 1.0 / P, None)
            comm.check()
            want = rs_reference(ins, P, n, 1.0 / P, torch.float32)
            for r in range(P):
                torch.testing.assert_close(outs[r], want[r], rtol=2e-2, atol=2e-2)
    events, dropped = comm.trace()
    assert dropped == 0 and len(events) > 0
    assert {e["rank"] for e in events} == set(range(P))
    assert {"signal", "wait"} <= {e["op"] for e in events}
    assert {"all_gather", "reduce_scatter"} <= {e["collective"] for e in events}
    assert all(a["t_ns"] <= b["t_ns"] for a, b in zip(events, events[1:]))
    # per rank and lane, call numbers never go backwards
    last = {}
    for e in events:
        key = (e["rank"], e["lane"])
        assert e["call"] >= last.get(key, 0)
        last[key] = e["call"]
    assert comm.trace() == ([], 0)                      # reading empties it
    comm.set_debug(0.0, 0)
    comm.close()


def test_python_api_on_single_rank_world():
    """world == 1: every collective degenerates to a local copy / scale through the kernels."""
    comm = pccl.Communicator.emulated_world(1, device=0, heap_bytes=4 << 20, staging_bytes=1 << 20)
    g = comm.world_group
    x = rand(1001, torch.bfloat16, 1)
    out = torch.zeros_like(x)
    pccl._all_gather(out, x, g, use_pccl_cpp_backend=True)
    assert torch.equal(out, x)
    o32 = torch.zeros(1001, device=DEV)
    pccl._reduce_scatter(o32, x, g, use_pccl_cpp_backend=True, scale=0.5)
    torch.testing.assert_close(o32, x.float() * 0.5)
    y = x.clone()
    pccl._all_reduce(y, g, algorithm="auto", scale=2.0)
    torch.testing.assert_close(y.float(), x.float() * 2.0, rtol=8e-3, atol=1e-3)
    req = pccl._all_gather(out, x, g, async_op=True, use_pccl_cpp_backend=True)
    req.wait()
    pccl.barrier(g)
    comm.check()


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("algo", [sch.RING, sch.RECURSIVE])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_all_reduce_as_reduce_scatter_plus_all_gather_in_one_launch(P, algo, dtype):
    """The reference's composition (recursive halving + doubling, or ring + ring) as one kernel:
    private tensors (staged) and symmetric tensors (zero-copy), several sizes, back to back."""
    comm = emu(P)
    gid = comm.world_group.gid
    for n in [P, 8 * P, 1000 * P, P * ((1 << 16) + 3)]:
        ts = [rand(n, dtype, 13 * r + n) for r in range(P)]
        want = sum(t.float() for t in ts) * 0.5
        comm.native.all_reduce(gid, ts, sch.ALGO_IDS[algo], 4, 0.5)
        comm.check()
        for r in range(P):
            # bf16 partial sums are rounded once per step of the schedule (up to P-1 times on the ring)
            tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else \
                dict(rtol=3e-2, atol=2e-2 * float(want.abs().max()) + 1e-3)
            torch.testing.assert_close(ts[r].float(), want, **tol)
            assert torch.equal(ts[r], ts[0]), "all ranks must hold bit-identical results"
    n = P * 5000
    sym = comm.empty(n, dtype)
    vals = [rand(n, dtype, 77 + r) for r in range(P)]
    for rep in range(2):
        for r in range(P):
            sym[r].copy_(vals[r])
        comm.native.all_reduce(gid, sym, sch.ALGO_IDS[algo], 3, 1.0)
        comm.check()
        want = sum(v.float() for v in vals)
        for r in range(P):
            tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else \
                dict(rtol=3e-2, atol=2e-2 * float(want.abs().max()) + 1e-3)
            torch.testing.assert_close(sym[r].float(), want, **tol)
    del sym
    # a count that the group size does not divide falls back to the two-shot kernel in the Python layer
    if P > 2:
        g = comm.world_group
        assert g.size == P


BIG = 9 * (1 << 20) + 24          # elements: > 1 MiB per lane on 4-7 lanes, odd tail, 16-byte aligned start


@pytest.mark.parametrize("P", [2, 4])
def test_copy_engine_paths_carry_bf16(P):
    """Sizes that give every lane more than a megabyte: bf16 data then goes through the copy-engine
    ring (cp.async.bulk) of every collective, which the small cases above never reach: all-gather
    direct with several destinations, reduce-scatter pull and the final step of the push variants
    (bf16 -> bf16 and bf16 -> fp32), all-reduce.  Against fp32 PyTorch sums."""
    comm = pccl.Communicator.emulated_world(P, device=0, heap_bytes=(P + 2) * BIG * 2 * 2 + (96 << 20), staging_bytes=P * BIG * 2 + (8 << 20))
    gid = comm.world_group.gid
    n = BIG
    # all-gather, symmetric output (zero-copy) and private output
    sym_out = comm.empty(P * n, torch.bfloat16)
    vals = [rand(n, torch.bfloat16, 5 + r) for r in range(P)]
    want = torch.cat(vals)
    for algo in (sch.DIRECT, sch.RING, sch.PULL):
        for r in range(P):
            sym_out[r].zero_()
        comm.native.all_gather(gid, sym_out, vals, sch.ALGO_IDS[algo], 6)
        comm.check()
        for r in range(P):
            assert torch.equal(sym_out[r], want), f"all_gather {algo} rank {r}"
    priv = [torch.zeros(P * n, dtype=torch.bfloat16, device=DEV) for _ in range(P)]
    comm.native.all_gather(gid, priv, vals, sch.ALGO_IDS[sch.DIRECT], 7)
    comm.check()
    for r in range(P):
        assert torch.equal(priv[r], want)
    del sym_out, priv
    # reduce-scatter: pull from symmetric inputs, push variants from private inputs
    m = n // P // 8 * 8
    sym_in = comm.empty(P * m, torch.bfloat16)
    ins = [rand(P * m, torch.bfloat16, 40 + r) for r in range(P)]
    for r in range(P):
        sym_in[r].copy_(ins[r])
    for tout in (torch.bfloat16, torch.float32):
        wantr = rs_reference(ins, P, m, 1.0 / P, tout)
        outs = [torch.zeros(m, dtype=tout, device=DEV) for _ in range(P)]
        comm.native.reduce_scatter(gid, outs, sym_in, sch.ALGO_IDS[sch.PULL], 4, 1.0 / P, None)
        comm.check()
        for r in range(P):
            tol = dict(rtol=1e-5, atol=1e-5) if tout == torch.float32 else dict(rtol=8e-3, atol=1e-5)
            torch.testing.assert_close(outs[r].float(), wantr[r].float(), **tol)
        for algo in (sch.DIRECT, sch.RING):
            outs = [torch.zeros(m, dtype=tout, device=DEV) for _ in range(P)]
            comm.native.reduce_scatter(gid, outs, ins, sch.ALGO_IDS[algo], 4, 1.0 / P, None)
            comm.check()
            for r in range(P):
                tol = dict(rtol=3e-2, atol=3e-2) if algo == sch.RING else \
                    (dict(rtol=1e-5, atol=1e-5) if tout == torch.float32 else dict(rtol=8e-3, atol=1e-5))
                torch.testing.assert_close(outs[r].float(), wantr[r].float(), **tol)
    del sym_in
    # all-reduce, private tensors, two-shot and two-phase
    for algo in (sch.DIRECT, sch.RING):
        ts = [rand(P * m, torch.bfloat16, 90 + r) for r in range(P)]
        want_ar = sum(t.float() for t in ts)
        comm.native.all_reduce(gid, ts, sch.ALGO_IDS[algo], 4, 1.0)
        comm.check()
        for r in range(P):
            torch.testing.assert_close(ts[r].float(), want_ar, rtol=3e-2, atol=2e-2 * float(want_ar.abs().max()))
    comm.close()


def test_collectives_of_different_groups_share_the_staging_area_in_order():
    """Two groups of one communicator use the same staging bytes.  An asynchronous all-gather on
    group A (side stream, private output: staged) followed at once by a reduce-scatter on group B
    (current stream, push variant: staged) must not overlap on a rank; both results are checked."""
    comm = pccl.Communicator.emulated_world(4, device=0, heap_bytes=64 << 20, staging_bytes=16 << 20)
    ga = comm.world_group
    gb = comm.new_group([0, 1, 2, 3])
    n = 300000
    side = torch.cuda.Stream(device=0)
    for rep in range(3):
        ins = [rand(n, torch.float32, rep * 10 + r) for r in range(4)]
        outs = [torch.zeros(4 * n, device=DEV) for _ in range(4)]
        big = [rand(4 * n, torch.float32, 50 + rep * 10 + r) for r in range(4)]
        red = [torch.zeros(n, device=DEV) for _ in range(4)]
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            comm.native.all_gather(ga.gid, outs, ins, sch.ALGO_IDS[sch.RING], 4)
        comm.native.reduce_scatter(gb.gid, red, big, sch.ALGO_IDS[sch.DIRECT], 4, 1.0, None)
        torch.cuda.synchronize()
        comm.check()
        want = rs_reference(big, 4, n, 1.0, torch.float32)
        for r in range(4):
            assert torch.equal(outs[r], torch.cat(ins)), f"all_gather rep {rep} rank {r}"
            torch.testing.assert_close(red[r], want[r], rtol=1e-5, atol=1e-5)
    comm.close()


def test_guard_words_and_extent_checks():
    """Debug aids that stand in for a memory checker: canary bytes around symmetric tensors, verified
    on the host, and a host-side check that every landing zone a launch names lies inside the heap."""
    comm = pccl.Communicator.emulated_world(4, device=0, heap_bytes=32 << 20, staging_bytes=4 << 20)
    comm.set_debug(guards=True)
    gid = comm.world_group.gid
    n = 12345
    outs = comm.empty(4 * n, torch.bfloat16)
    sym_in = comm.empty(4 * n, torch.bfloat16)
    vals = [rand(n, torch.bfloat16, 3 + r) for r in range(4)]
    for algo in (sch.DIRECT, sch.RING, sch.RECURSIVE, sch.PULL):
        comm.native.all_gather(gid, outs, vals, sch.ALGO_IDS[algo], 5)
    for r in range(4):
        sym_in[r].copy_(rand(4 * n, torch.bfloat16, 40 + r))
    res = [torch.zeros(n, device=DEV) for _ in range(4)]
    for algo in (sch.DIRECT, sch.RING, sch.RECURSIVE, sch.PULL):
        comm.native.reduce_scatter(gid, res, sym_in, sch.ALGO_IDS[algo], 5, 1.0, None)
    comm.native.all_reduce(gid, outs, sch.ALGO_IDS[sch.RING], 4, 1.0)
    comm.check()
    comm.check_guards()                                   # nothing wrote outside its buffer
    assert torch.equal(outs[0], outs[3])
    # a stray write just behind a buffer is found and attributed
    off = comm.native.offset_of(outs[2].data_ptr(), outs[2].numel() * 2, 2)
    comm.native.tensor(off + 4 * n * 2 + 7, 1, torch.uint8, 2).fill_(0)
    with pytest.raises(pccl.PcclError, match="behind"):
        comm.check_guards()
    # a landing zone that leaves the heap is refused before anything is launched
    with pytest.raises(RuntimeError, match="leaves the symmetric heap"):
        ag2d_outer_call(comm.native, gid, sch.ALGO_IDS[sch.RING], 2, [v.data_ptr() for v in vals], (32 << 20) - 1000, 0,
                        n * 2, 1)
    comm.check()
    comm.close()


@pytest.mark.parametrize("P", [2, 4, 8])
def test_eager_small_messages(P):
    """The handshake-free variant for small messages on the world group: direct schedule into the
    alternating halves of the communicator's eager area.  Back-to-back calls of changing size (and
    lane count), all-gather and reduce-scatter mixed, private and symmetric tensors, with stress
    jitter: the halves must never be overwritten while a slower rank still reads them."""
    comm = pccl.Communicator.emulated_world(P, device=0, heap_bytes=64 << 20, staging_bytes=8 << 20)
    gid = comm.world_group.gid
    cap = comm.native.eager_capacity
    assert cap >= 1 << 20
    E = sch.ALGO_IDS[sch.EAGER]
    sym_out = comm.empty(P * 70000, torch.bfloat16)
    for jitter in (0.0, 120.0):
        comm.set_debug(jitter_us=jitter)
        for rep, n in enumerate([1, 17, 4099, 70000, 33, 65536, 5]):
            lanes = 1 + rep % 5
            ins = [rand(n, torch.bfloat16, 1000 * rep + r) for r in range(P)]
            outs = [torch.zeros(P * n, dtype=torch.bfloat16, device=DEV) for _ in range(P)] if rep % 2 == 0 else \
                [t[:P * n] for t in sym_out]
            comm.native.all_gather(gid, outs, ins, E, lanes)
            big = [rand(P * n, torch.bfloat16, 7000 * rep + r) for r in range(P)]
            res = [torch.zeros(n, dtype=torch.float32, device=DEV) for _ in range(P)]
            comm.native.reduce_scatter(gid, res, big, E, lanes, 1.0 / P, None)
            comm.check()
            want = torch.cat(ins)
            want_rs = rs_reference(big, P, n, 1.0 / P, torch.float32)
            for r in range(P):
                assert torch.equal(outs[r], want), f"eager all_gather P={P} n={n} rank {r}"
                torch.testing.assert_close(res[r], want_rs[r], rtol=1e-5, atol=1e-5)
    comm.set_debug(0.0, 0)
    too_big = cap // P // 2 + 8
    with pytest.raises(RuntimeError, match="eager area"):
        comm.native.all_gather(gid, [torch.zeros(P * too_big, dtype=torch.bfloat16, device=DEV) for _ in range(P)],
                               [torch.zeros(too_big, dtype=torch.bfloat16, device=DEV) for _ in range(P)], E, 2)
    del sym_out
    comm.close()
