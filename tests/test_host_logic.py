"""Host-side logic that needs neither a GPU nor several processes: the tuner, the engine's
region layout, request handles and the single-process side of the API."""
import pytest
import torch

from pccl import schedule as sch
from pccl import tuner
from pccl.models.gpt import PRESETS, GPTConfig, unit_specs
from pccl.parallel.zero3 import heap_bytes_needed, unit_regions
from pccl.request import Request


def test_tuner_picks_first_feasible_variant():
    # small all-gather at P=8: NVLS when there is a multicast mapping and a symmetric output, else direct
    assert tuner.choose("all_gather", 8, 1 << 20, symmetric_out=True, has_multimem=True)[0] == sch.MULTIMEM
    assert tuner.choose("all_gather", 8, 1 << 20, symmetric_out=True, has_multimem=False)[0] == sch.DIRECT
    assert tuner.choose("all_gather", 8, 1 << 20, symmetric_out=False, has_multimem=True)[0] == sch.DIRECT
    assert tuner.choose("all_gather", 8, 512 << 20, symmetric_out=True, has_multimem=True)[0] == sch.DIRECT
    # reduce-scatter: pull needs the input in the heap; private inputs fall through to a push schedule
    assert tuner.choose("reduce_scatter", 8, 256 << 20, symmetric_in=True)[0] == sch.PULL
    assert tuner.choose("reduce_scatter", 8, 256 << 20, symmetric_in=False)[0] == sch.RING
    assert tuner.choose("reduce_scatter", 8, 8 << 20, symmetric_in=False)[0] == sch.RECURSIVE
    # a group size without a table row still works
    assert tuner.choose("reduce_scatter", 6, 8 << 20)[0] == sch.DIRECT


def test_tuner_explicit_requests_and_lanes(monkeypatch):
    algo, lanes = tuner.choose("all_gather", 4, 64 << 20, requested=sch.RING, lanes=7)
    assert (algo, lanes) == (sch.RING, 7)
    with pytest.raises(ValueError):
        tuner.choose("all_gather", 6, 1 << 20, requested=sch.RECURSIVE)       # asked for explicitly: refuse, do not swap
    assert tuner.choose("reduce_scatter", 8, 1 << 20, requested=sch.PULL, symmetric_in=False)[0] == sch.DIRECT
    assert tuner.choose("all_gather", 8, 4096, max_lanes=148)[1] == 1         # tiny messages use one lane
    assert tuner.choose("all_gather", 8, 1 << 30, max_lanes=148)[1] == 64
    monkeypatch.setenv("PCCL_ALGO", "ring")
    monkeypatch.setenv("PCCL_LANES", "3")
    assert tuner.choose("all_gather", 8, 1 << 20) == (sch.RING, 3)


def test_unit_regions_cover_the_unit_and_shard_evenly():
    for name in ("gpt-1.3b", "gpt-7b"):
        cfg = PRESETS[name]
        layer = unit_specs(cfg)[1]
        for world in (1, 2, 4, 8):
            plain = unit_regions(layer, world, False)
            assert len(plain) == 1 and plain[0][0] == 0 and plain[0][1] >= layer.numel and plain[0][1] % (256 * world) == 0
            fused = unit_regions(layer, world, True)
            assert [r[0] for r in fused][:2] == [0, 3 * cfg.d_model * cfg.d_model]
            assert fused[0][1] == 3 * cfg.d_model * cfg.d_model and fused[1][1] == cfg.d_ff * cfg.d_model
            end = 0
            for off, length in fused:
                assert off == end and length % (256 * world) == 0
                end = off + length
            assert end >= layer.numel
        embed = unit_specs(cfg)[0]
        assert len(unit_regions(embed, 8, True)) == 1          # only the blocks have row-sharded weights
    assert heap_bytes_needed(PRESETS["gpt-1.3b"], 8) < heap_bytes_needed(PRESETS["gpt-1.3b"], 1)


def test_model_sizes_match_the_benchmark_configurations():
    assert abs(PRESETS["gpt-1.3b"].num_params() / 1e9 - 1.316) < 0.01
    assert abs(PRESETS["gpt-7b"].num_params() / 1e9 - 6.66) < 0.02
    cfg = GPTConfig(2, 256, 4, 1024, vocab=1024, seq_len=128)
    names = [p.name for p in unit_specs(cfg)[1].params]
    assert names[:2] == ["qkv_w", "fc1_w"]                       # the fused kernel relies on this order
    for u in unit_specs(cfg):
        for p in u.params:
            assert p.offset % 256 == 0


def test_request_wraps_handles_and_runs_the_epilogue():
    class Done:
        _pccl_completed = True

    seen = []
    r = Request(Done())
    assert r.backend == "completed" and r.is_completed()
    assert r.wait(lambda: seen.append("x")) is None and seen == ["x"]
    with pytest.raises(TypeError):
        r.wait(epilogue=3)
    with pytest.raises(ValueError):
        Request(object())
    assert "completed" in repr(r)


def test_group_type_is_checked():
    import pccl

    with pytest.raises(TypeError):
        pccl._all_gather(torch.empty(4), torch.empty(2), group="not a group")
    with pytest.raises(TypeError):
        pccl._reduce_scatter(torch.empty(2), torch.empty(4), group=42)
    with pytest.raises(TypeError):
        pccl._all_reduce(torch.empty(2), group=3.5)
