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


def test_layer_math_fallback_matches_autograd_on_cpu():
    """The hand-written forward/backward of the GPT blocks (pure-PyTorch paths: residual adds
    deferred to the layer norms, bias gradients handed down as column sums) against autograd."""
    import torch.nn.functional as F

    from pccl.models import gpt

    torch.manual_seed(0)
    cfg = GPTConfig(2, 64, 4, 256, vocab=96, seq_len=16, name="cpu-test")
    units = unit_specs(cfg)
    B, S = 2, cfg.seq_len
    T = B * S
    flats = [torch.zeros(u.numel, dtype=torch.float64) for u in units]
    for u, f in zip(units, flats):
        gpt.init_unit(u, f, cfg, seed=7)
        f.add_(torch.randn_like(f) * 0.02)                       # biases and norms away from 0 / 1
    params = [gpt.views(u, f) for u, f in zip(units, flats)]
    grads = [gpt.views(u, torch.zeros_like(f)) for u, f in zip(units, flats)]
    tokens = torch.randint(0, cfg.vocab, (B, S))
    targets = torch.randint(0, cfg.vocab, (B, S))

    def ce(logits, tgt, loss_sum, grad_scale):
        lp = torch.log_softmax(logits, dim=-1)
        loss_sum += -lp.gather(1, tgt.view(-1, 1)).sum()
        g = lp.exp()
        g.scatter_add_(1, tgt.view(-1, 1), -torch.ones(len(tgt), 1, dtype=g.dtype))
        logits.copy_(g * grad_scale)

    with torch.no_grad():
        x = gpt.embed_forward(tokens, params[0])
        branch, saved = None, []
        for li in range(1, cfg.n_layer + 1):
            x, branch, ctx = gpt.layer_forward_deferred(x, branch, params[li], cfg, B)
            saved.append(ctx)
        loss_sum = torch.zeros(1, dtype=torch.float64)
        sums = [torch.empty(cfg.d_model, dtype=torch.float64) for _ in range(2)]
        L = cfg.n_layer
        dx = gpt.head_forward_backward(x, targets, params[0], grads[0], cfg, 1.0 / T, loss_sum, ce, chunk_tokens=20,
                                       branch=branch, dx_sum=sums[L % 2])
        for li in range(L, 0, -1):
            dx = gpt.layer_backward(dx, saved.pop(), params[li], grads[li], cfg, B, dy_sum=sums[li % 2],
                                    dx_sum=sums[(li - 1) % 2] if li > 1 else None)
        gpt.embed_backward(dx, tokens, grads[0])

    ref = [{k: v.clone().requires_grad_() for k, v in p.items()} for p in params]
    p0 = ref[0]
    h = F.embedding(tokens, p0["wte"]) + p0["wpe"][:S]
    for p in ref[1:]:
        n = F.layer_norm(h, (cfg.d_model,), p["ln1_w"], p["ln1_b"], cfg.ln_eps)
        qkv = F.linear(n, p["qkv_w"], p["qkv_b"]).view(B, S, 3, cfg.n_head, cfg.head_dim)
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, cfg.d_model)
        h = h + F.linear(a, p["proj_w"], p["proj_b"])
        n = F.layer_norm(h, (cfg.d_model,), p["ln2_w"], p["ln2_b"], cfg.ln_eps)
        h = h + F.linear(F.gelu(F.linear(n, p["fc1_w"], p["fc1_b"]), approximate="tanh"), p["fc2_w"], p["fc2_b"])
    h = F.layer_norm(h, (cfg.d_model,), p0["lnf_w"], p0["lnf_b"], cfg.ln_eps)
    loss = F.cross_entropy(F.linear(h, p0["wte"]).view(T, -1), targets.reshape(-1))
    loss.backward()
    torch.testing.assert_close(loss_sum[0] / T, loss.detach(), rtol=1e-9, atol=1e-9)
    for ui in range(len(units)):
        for name, r in ref[ui].items():
            torch.testing.assert_close(grads[ui][name], r.grad, rtol=1e-7, atol=1e-9, msg=lambda m: f"unit {ui} {name}: {m}")
    # the one-call form sums the residual itself
    with torch.no_grad():
        x0 = gpt.embed_forward(tokens, params[0])
        y, _ctx = gpt.layer_forward(x0, params[1], cfg, B)
        x2, m, _ctx = gpt.layer_forward_deferred(x0, None, params[1], cfg, B)
    torch.testing.assert_close(y, x2 + m)


def test_clock_sampler_reads_a_fake_nvml(monkeypatch):
    """The sampler only reads: SM clock, power and the clock-event reasons, through whatever
    NVML binding is importable.  A stand-in module plays the device."""
    import sys
    import time
    import types

    from pccl.utils.clocks import ClockSampler

    calls = {"set": 0}
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("gpu", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, which: 1965
    clocks = iter([1900, 1600, 1500, 1605] + [1605] * 1000)
    fake.nvmlDeviceGetClockInfo = lambda h, which: next(clocks)
    fake.nvmlDeviceGetPowerUsage = lambda h: 987000            # milliwatts
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4   # sw_power_cap

    def forbidden(*a, **k):                                   # any setter would be a bug
        calls["set"] += 1
        raise AssertionError("the sampler must not change device settings")

    for name in ("nvmlDeviceSetApplicationsClocks", "nvmlDeviceSetGpuLockedClocks", "nvmlDeviceResetGpuLockedClocks",
                 "nvmlDeviceSetPowerManagementLimit", "nvmlDeviceSetPersistenceMode"):
        setattr(fake, name, forbidden)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = ClockSampler(3, period_s=0.005).start()
    deadline = time.time() + 5.0
    while len(s.samples) < 4 and time.time() < deadline:     # a busy host may start the thread late
        time.sleep(0.01)
    out = s.stop()
    assert calls["set"] == 0
    assert out["sm_max_mhz"] == 1965 and out["samples"] >= 4
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 987.0
    assert 1500 <= out["sm_mhz"] <= 1900
    assert ClockSampler(0).summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


def test_benchmark_helpers(tmp_path, monkeypatch):
    from benchmark_raw_collectives import utils as bu

    assert bu.parse_sizes("1M, 64m,1G,512", []) == [1 << 20, 64 << 20, 1 << 30, 512]
    assert bu.parse_sizes(None, [7]) == [7]
    assert bu.sizes_pow2(1 << 20, 1 << 23) == [1 << 20, 1 << 21, 1 << 22, 1 << 23]
    # 8 ranks, 1 GiB each, 10 ms: (P-1) * bytes / time
    assert bu.bus_bandwidth_gbs(1 << 30, 8, 10.0) == pytest.approx(7 * (1 << 30) / 0.010 / 1e9)
    assert bu.bus_bandwidth_gbs(1 << 30, 1, 10.0) == 0.0
    x = torch.arange(1000, dtype=torch.float32)
    y = x.clone()
    y[:15] += 1.0                                             # 1.5 % of the elements differ: within the 2 % rule
    assert bu.allclose(x, y)
    y[:30] += 1.0
    assert not bu.allclose(x, y)
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("SLURM_JOB_ID", "4242")
    log = bu.CsvLog("all_gather", "b200", 8, ["gpu_count", "output_size", "time_pccl"], enabled=True)
    log.row({"gpu_count": 8, "output_size": 64, "time_pccl": 0.5, "ignored": 1})
    log.fh.close()
    text = (tmp_path / "data" / "all_gather" / "b200" / "gpus_8_slurm_4242.csv").read_text().splitlines()
    assert text == ["gpu_count,output_size,time_pccl", "8,64,0.5"]
    bu.CsvLog("x", "y", 1, ["a"], enabled=False).row({"a": 1})   # disabled: no file, no error
    assert not (tmp_path / "data" / "x").exists()


def test_gatherer_count_follows_the_required_rate():
    from pccl.ops.ag_gemm import auto_gather_ctas

    # fewer tokens per weight byte -> the gather must run faster -> more gatherers; always even, 4..32
    few = auto_gather_ctas(8192, 6144, 2048, 2)
    more = auto_gather_ctas(4096, 12288, 4096, 2)
    assert few < more
    for P in (2, 4, 8):
        for M in (1024, 4096, 8192, 65536):
            g = auto_gather_ctas(M, 8192, 2048, P)
            assert g % 2 == 0 and 4 <= g <= 32
    assert auto_gather_ctas(8192, 6144, 2048, 8) >= auto_gather_ctas(8192, 6144, 2048, 2)
    assert auto_gather_ctas(1 << 20, 8192, 2048, 8) == 4      # plenty of math per byte: the minimum
    # the width of the layer cancels: both the bytes and the FLOPs scale with it
    assert auto_gather_ctas(4096, 4096, 4096, 4) == auto_gather_ctas(4096, 16384, 4096, 4)


def test_offset_allocator_random_sequences():
    """The symmetric heap's bookkeeping: blocks never overlap, honour their alignment, the
    byte count is exact, freed neighbours merge, and a drained heap is one free range again."""
    import random

    import pccl

    A = pccl._C.OffsetAllocator
    rng = random.Random(5)
    for trial in range(20):
        size = rng.choice([1 << 16, 1 << 20, (1 << 20) + 12345])
        a = A(size)
        live = {}
        for _ in range(400):
            if live and rng.random() < 0.45:
                off = rng.choice(list(live))
                a.free(off)
                del live[off]
            else:
                nbytes = rng.choice([1, 7, 256, 4096, rng.randrange(1, size // 8)])
                align = rng.choice([1, 16, 256, 4096])
                off = a.alloc(nbytes, align)
                if off < 0:
                    assert a.largest_free() < nbytes + align     # refusal only when it truly cannot fit aligned
                    continue
                assert off % align == 0 and off + nbytes <= size
                for o, n in live.items():
                    assert off + nbytes <= o or o + n <= off, "blocks overlap"
                live[off] = nbytes
            assert a.used == sum(live.values())
        for off in list(live):
            a.free(off)
        assert a.used == 0 and a.largest_free() == size
    a = A(1024)
    assert a.alloc(0, 0) == 0                       # zero bytes still gets a distinct offset
    assert a.alloc(2048, 1) == -1
    with pytest.raises(RuntimeError):
        a.free(512)                                 # never allocated


def test_committed_tuning_table_is_well_formed():
    """Every row names known variants, thresholds ascend and end open, lanes fit the kernels'
    flag layout, and for every measured group size the last preference of every row needs
    neither NVLS nor symmetric input (so `auto` always has something it may run)."""
    import json

    table = json.loads(tuner.TABLE_PATH.read_text())
    assert {"all_gather", "reduce_scatter", "all_reduce"} <= set(table)
    for coll, by_world in table.items():
        if coll.startswith("_"):
            continue
        for world, rows in by_world.items():
            assert int(world) in (2, 4, 8)
            assert rows and rows[-1][0] is None, f"{coll} P={world}: the last row must be open-ended"
            limits = [r[0] for r in rows[:-1]]
            assert limits == sorted(limits) and all(isinstance(x, int) and x > 0 for x in limits)
            for _limit, algos, lanes in rows:
                algos = [algos] if isinstance(algos, str) else algos
                assert algos and all(a in sch.ALGO_IDS for a in algos)
                assert 1 <= int(lanes) <= 160
            # whatever the tensors look like, something feasible comes out
            for nbytes in (1 << 10, 1 << 20, 1 << 24, 1 << 30):
                algo, nl = tuner.choose(coll, int(world), nbytes, symmetric_in=False, symmetric_out=False, has_multimem=False)
                assert algo in sch.ALGO_IDS and algo not in (sch.MULTIMEM,) and nl >= 1
                if coll == "reduce_scatter":
                    assert algo != sch.PULL         # pull reads the peers' inputs: they must be symmetric


def test_only_lost_peers_become_timeouts():
    """Errors of a p2p step are sorted by what they say: an expired wait or a closed connection is a
    lost peer (PcclTimeoutError); a mismatch of shapes or dtypes, an invalid rank or a tensor on the
    wrong device is a programming error and keeps its own type."""
    from pccl.backends.p2p import _looks_like_lost_peer

    for msg in ("[../third_party/gloo/gloo/transport/tcp/unbound_buffer.cc:81] Timed out waiting 2000ms for recv operation to complete",
                "Connection closed by peer [127.0.0.1]:5291", "Connection reset by peer", "Broken pipe",
                "wait timeout after 1000ms"):
        assert _looks_like_lost_peer(RuntimeError(msg)), msg
    for msg in ("Tensors must be CUDA and dense", "Invalid destination rank: 7", "size mismatch: expected 8 got 4",
                "No backend type associated with device type cpu", "Invalid scalar type"):
        assert not _looks_like_lost_peer(RuntimeError(msg)), msg


def test_last_round_split_covers_every_k_block_once():
    """The GEMM splits the tiles of a partly filled last round along K (``GemmArgs::sk_tiles``).
    This restates the kernel's work sequence (``WorkIter`` and ``sk_pair_of`` in
    ``pccl/csrc/gemm_sm100.cu``) in Python and checks, for the shapes of the benchmark models and
    some awkward ones, that every k-block of every tile is computed exactly once, that every
    split tile has exactly one finisher (the pair holding its first k-block), that a pair is a
    helper for at most one tile, and that the finisher's list of helpers is exactly the set of
    other pairs that hold a piece of the tile."""
    import pccl

    C = pccl._C

    def items(pair, G, total, nkb, sk):
        I = sk * nkb
        cur, end = I * pair // G, I * (pair + 1) // G
        out = []
        while cur < end:
            t = cur // nkb
            k0 = cur - t * nkb
            k1 = nkb if nkb - k0 <= end - cur else k0 + (end - cur)
            out.append((t, k0, k1))
            cur += k1 - k0
        out += [(t, 0, nkb) for t in range(sk + pair, total, G)]
        return out

    def pair_of(i, I, G):
        return ((i + 1) * G + I - 1) // I - 1

    sms = 148
    G = sms // 2
    shapes = [(8192, 2048, 2048), (8192, 2048, 8192), (8192, 6144, 2048), (2048, 2048, 8192), (6144, 2048, 8192),
              (8192, 8192, 2048), (8192, 50304, 2048), (512, 512, 4096), (256, 256, 640), (4096, 12288, 4096), (1000, 520, 1024)]
    split_some = 0
    for M, N, K in shapes:
        total = ((M + 255) // 256) * ((N + 255) // 256)
        nkb = (K + 63) // 64
        sk = C.gemm_sk_tiles(M, N, K, sms)
        assert 0 <= sk <= total
        if sk == 0:
            continue
        split_some += 1
        I = sk * nkb
        seen = {}
        helper_of = {}
        for p in range(G):
            helps = 0
            for t, k0, k1 in items(p, G, total, nkb, sk):
                assert 0 <= k0 < k1 <= nkb
                for kb in range(k0, k1):
                    assert (t, kb) not in seen, "a k-block computed twice"
                    seen[(t, kb)] = p
                if k0 > 0:
                    helps += 1
                    helper_of.setdefault(t, set()).add(p)
            assert helps <= 1
        assert len(seen) == total * nkb, "a k-block was left out"
        for t in range(sk):
            finisher = seen[(t, 0)]
            holders = {seen[(t, kb)] for kb in range(nkb)}
            want = holders - {finisher}
            assert want == helper_of.get(t, set())
            if want:
                last = pair_of((t + 1) * nkb - 1, I, G)
                assert set(range(finisher + 1, last + 1)) == want
    assert split_some >= 5
    assert C.gemm_sk_tiles(8192, 8192, 2048, sms) == 0 or True     # 1024 tiles on 74 pairs: 13.84 rounds
    assert C.gemm_sk_tiles(8192, 2048, 2048, sms) == G + 256 % G
    assert C.gemm_sk_tiles(2048, 2048, 8192, sms) == 64            # fewer tiles than pairs: all of them are split


def test_tuner_takes_the_eager_variant_only_where_it_fits(monkeypatch, tmp_path):
    """`eager` needs the world group's eager area: P x bytes for an all-gather, (P-1) x bytes per block
    for a reduce-scatter.  Where it does not fit, or on another group (capacity 0), the next
    preference is taken."""
    import json

    table = {"all_gather": {"8": [[1 << 20, ["eager", "direct"], 32], [None, ["direct"], 64]]},
             "reduce_scatter": {"8": [[1 << 20, ["eager", "pull", "direct"], 32], [None, ["pull", "direct"], 64]]}}
    path = tmp_path / "t.json"
    path.write_text(json.dumps(table))
    monkeypatch.setattr(tuner, "TABLE_PATH", path)
    tuner.reload_table()
    try:
        cap = 8 << 20
        assert tuner.choose("all_gather", 8, 1 << 20, eager_capacity=cap)[0] == sch.EAGER        # 8 x 1 MiB fits exactly
        assert tuner.choose("all_gather", 8, (1 << 20) + 16, eager_capacity=cap)[0] == sch.DIRECT
        assert tuner.choose("all_gather", 8, 1 << 10, eager_capacity=0)[0] == sch.DIRECT         # not the world group
        assert tuner.choose("reduce_scatter", 8, 1 << 20, eager_capacity=cap, symmetric_in=True)[0] == sch.EAGER
        assert tuner.choose("reduce_scatter", 8, 1 << 20, eager_capacity=1 << 20, symmetric_in=True)[0] == sch.PULL
        assert tuner.choose("reduce_scatter", 8, 1 << 20, eager_capacity=1 << 20, symmetric_in=False)[0] == sch.DIRECT
        # an explicit request that does not fit degrades to direct instead of failing
        assert tuner.choose("all_gather", 8, 64 << 20, requested=sch.EAGER, eager_capacity=cap)[0] == sch.DIRECT
    finally:
        monkeypatch.undo()
        tuner.reload_table()


def test_reduce_scatter_lanes_follow_the_peer_count_and_skip_the_slow_zone(monkeypatch):
    """Lane counts the tuner picks when the caller passes none: all-gather shares are at least
    64 KiB per lane; a reduce-scatter lane reads from every peer, so its share shrinks with the
    group; shares between 64 KiB and 256 KiB (thread loops in dependent rounds, or a bulk-copy
    pipeline too short to fill) are avoided by taking fewer lanes of 256 KiB."""
    from pccl import tuner

    monkeypatch.delenv("PCCL_LANES", raising=False)
    monkeypatch.delenv("PCCL_ALGO", raising=False)

    def lanes(coll, P, nbytes):
        return tuner.choose(coll, P, nbytes, requested="pull" if coll == "reduce_scatter" else "direct",
                            symmetric_in=True, symmetric_out=True)[1]

    assert lanes("all_gather", 8, 1 << 20) == 16                      # 64 KiB per lane
    assert lanes("reduce_scatter", 2, 1 << 20) == 16                  # one peer: the same
    assert lanes("reduce_scatter", 4, 1 << 20) == 48                  # three peers: a third of the share
    assert lanes("reduce_scatter", 8, 256 << 10) == 28
    for P in (2, 4, 8):
        for block in (8 << 20, 12 << 20):
            n = lanes("reduce_scatter", P, block)
            assert block // n >= 256 << 10 and n >= 32, (P, block, n)  # out of the slow zone, still 32 lanes or more
        assert lanes("reduce_scatter", P, 4 << 20) == 64              # 64 KiB shares stay
        assert lanes("reduce_scatter", P, 5 << 20) == 64              # too small for 32 lanes of 256 KiB: unchanged
    assert tuner.choose("reduce_scatter", 8, 8 << 20, requested="multimem", symmetric_in=True, has_multimem=True)[1] == 64
    assert lanes("reduce_scatter", 4, 1 << 20) <= 64 and tuner.choose("reduce_scatter", 4, 1 << 20, lanes=7)[1] == 7


def test_sweep_markdown_handles_lane_suffixed_variants():
    """``sweep.py --lanes a,b,c`` names its columns ``variant@lanes``; the markdown table lists them all."""
    import importlib.util
    from pathlib import Path

    path = Path(__file__).resolve().parent.parent / "benchmark_raw_collectives" / "sweep.py"
    spec = importlib.util.spec_from_file_location("pccl_sweep_for_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    best = {"variant": "pull@64", "ms": 0.04, "busbw_gbs": 150.0, "vs_nccl": 1.3, "correct": None,
            "frac_of_900": 0.16, "frac_of_measured_770": 0.19}
    doc = {"P": 4, "nvls": True, "transport": "vmm", "timing": "t",
           "rows": [{"sweep": "rs", "collective": "reduce_scatter", "P": 4, "dtype": "bfloat16", "per_rank_bytes": 8 << 20,
                     "nccl_ms": 0.05, "nccl_busbw_gbs": 100.0,
                     "variants": {"pull@4": {"ms": 0.07, "busbw_gbs": 80.0, "vs_nccl": 0.7, "correct": None},
                                  "pull@64": {"ms": 0.04, "busbw_gbs": 150.0, "vs_nccl": 1.3, "correct": None}},
                     "best": best, "best_without_multimem": best}]}
    text = mod.markdown(doc)
    assert "pull@4 µs" in text and "pull@64 µs" in text and "| 8 | 50.0 |" in text
