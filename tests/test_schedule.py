"""Schedules simulated for all P ranks in one process: no GPU, no processes."""
import numpy as np
import pytest

from pccl import schedule as sch

ALGOS = [sch.DIRECT, sch.RING, sch.RECURSIVE]


def worlds(algo):
    return [1, 2, 4, 8] if algo == sch.RECURSIVE else [1, 2, 3, 4, 5, 6, 7, 8]


@pytest.mark.parametrize("algo", ALGOS)
def test_all_gather_schedule_delivers_every_block(algo):
    for P in worlds(algo):
        have = [{r} for r in range(P)]
        for t in range(sch.num_steps(algo, P)):
            steps = [sch.ag_step(algo, P, r, t) for r in range(P)]
            incoming = [set() for _ in range(P)]
            for r, s in enumerate(steps):
                # what I send is what my destination expects from me
                d = steps[s.dst]
                assert d.src == r and d.recv_first == s.send_first and d.nblocks == s.nblocks
                blocks = set(range(s.send_first, s.send_first + s.nblocks))
                assert blocks <= have[r], f"{algo} P={P} step {t}: rank {r} forwards blocks it does not hold"
                incoming[s.dst] |= blocks
            for r in range(P):
                assert not (incoming[r] & have[r]), "a block was delivered twice"
                have[r] |= incoming[r]
        for r in range(P):
            assert have[r] == set(range(P))


@pytest.mark.parametrize("algo", ALGOS)
def test_reduce_scatter_schedule_sums_every_block(algo):
    rng = np.random.default_rng(0)
    for P in worlds(algo):
        n = 3
        inputs = rng.standard_normal((P, P, n))
        nsteps = sch.num_steps(algo, P)
        staged = [dict() for _ in range(P)]   # rank -> {step: (recv_first, array[nblocks, n])}

        def partial(r, b, t):
            acc = inputs[r, b].copy()
            for j in sch.rs_dep_steps(algo, P, t):
                lo, arr = staged[r][j]
                if lo <= b < lo + arr.shape[0]:
                    acc += arr[b - lo]
            return acc

        total_slots = 0
        for t in range(nsteps):
            steps = [sch.rs_step(algo, P, r, t) for r in range(P)]
            payloads = []
            for r, s in enumerate(steps):
                d = steps[s.dst]
                assert d.src == r and d.recv_first == s.send_first and d.nblocks == s.nblocks
                payloads.append(np.stack([partial(r, b, t) for b in range(s.send_first, s.send_first + s.nblocks)]))
            for r, s in enumerate(steps):
                staged[s.dst][t] = (s.send_first, payloads[r])
            total_slots = max(total_slots, sch.rs_stage_offset(algo, P, t) + steps[0].nblocks)
        assert total_slots <= max(P - 1, 0)
        for r in range(P):
            np.testing.assert_allclose(partial(r, r, nsteps), inputs[:, r].sum(axis=0), rtol=1e-12, atol=1e-12)


def test_staging_slots_do_not_overlap():
    for algo in ALGOS:
        for P in worlds(algo):
            used = set()
            for t in range(sch.num_steps(algo, P)):
                s = sch.rs_step(algo, P, 0, t)
                off = sch.rs_stage_offset(algo, P, t)
                slots = set(range(off, off + s.nblocks))
                assert not (slots & used)
                used |= slots
            assert used == set(range(max(P - 1, 0)))


def test_recursive_matches_reference_description():
    # distance doubling for all-gather (nearest partner first), halving for reduce-scatter
    assert [sch.ag_step(sch.RECURSIVE, 8, 0, t).dst for t in range(3)] == [1, 2, 4]
    assert [sch.rs_step(sch.RECURSIVE, 8, 0, t).dst for t in range(3)] == [4, 2, 1]
    s = sch.ag_step(sch.RECURSIVE, 8, 5, 1)   # rank 5, seg 2: partner 7, holds blocks 4..5
    assert (s.dst, s.send_first, s.recv_first, s.nblocks) == (7, 4, 6, 2)
    s = sch.rs_step(sch.RING, 4, 1, 0)
    assert (s.dst, s.src, s.send_first, s.recv_first) == (2, 0, 0, 3)


def test_recursive_rejects_non_power_of_two():
    with pytest.raises(ValueError):
        sch.check_algo(sch.RECURSIVE, 6)
    sch.check_algo(sch.RING, 6)
    with pytest.raises(ValueError):
        sch.check_algo("bogus", 4)


def test_header_and_python_agree():
    """The device header (through the extension) and the Python twin, step by step."""
    pccl_C = pytest.importorskip("pccl.build_kernels").load()
    for name in ALGOS:
        a = sch.ALGO_IDS[name]
        for P in worlds(name):
            assert pccl_C.num_steps(a, P) == sch.num_steps(name, P)
            for t in range(sch.num_steps(name, P)):
                assert pccl_C.rs_stage_offset(a, P, t) == sch.rs_stage_offset(name, P, t)
                for r in range(P):
                    for cfn, pfn in ((pccl_C.ag_step, sch.ag_step), (pccl_C.rs_step, sch.rs_step)):
                        s = pfn(name, P, r, t)
                        assert cfn(a, P, r, t) == (s.dst, s.src, s.send_first, s.recv_first, s.nblocks)
            for t in range(sch.num_steps(name, P) + 1):
                mask = pccl_C.rs_dep_mask(a, P, t)
                assert [j for j in range(8) if (mask >> j) & 1] == sch.rs_dep_steps(name, P, t)


def test_grid_coords():
    assert sch.grid_coords(5, 2, 2) == (1, 0, 1)
    assert sch.grid_coords(3, 2, 2) == (0, 1, 1)
