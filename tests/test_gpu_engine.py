"""ZeRO-3 engine and training kernels on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_heap_blocks_do_not_overlap_and_are_recycled():
    import pccl

    comm = pccl.Communicator.emulated_world(2, device=0, heap_bytes=8 << 20, staging_bytes=1 << 20)
    a = comm.empty(1000, torch.float32)
    b = comm.empty(1000, torch.float32)
    pa, pb = a[0].data_ptr(), b[0].data_ptr()
    assert abs(pa - pb) >= 4000
    used = comm.native.heap_used
    view = a[0][10:20]
    del a
    assert comm.native.heap_used == used        # the view keeps the block alive
    del view
    assert comm.native.heap_used < used
    c = comm.empty(1000, torch.float32)
    assert c[0].data_ptr() == pa                # first fit reuses the freed block
    with pytest.raises(pccl.PcclError):
        comm.empty(1 << 30, torch.float32)


def test_adamw_matches_reference():
    import pccl

    C = pccl._C
    n = 100003
    g = torch.Generator(device=DEV).manual_seed(0)
    master = torch.randn(n, device=DEV, generator=g)
    grad = torch.randn(n, device=DEV, generator=g) * 3
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    param = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ref_p = master.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    sq = torch.zeros(1, device=DEV)
    for step in range(1, 4):
        sq.zero_()
        C.sq_norm(grad, sq)
        torch.testing.assert_close(sq, (grad.double() ** 2).sum().float().view(1), rtol=1e-4, atol=0)
        C.adamw(master, m, v, grad, param, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0, 1.0, sq)
        ref_p.grad = grad.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        torch.testing.assert_close(master, ref_p.detach(), rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(param.float(), master, rtol=8e-3, atol=1e-6)
    gb = grad.to(torch.bfloat16)
    sq.zero_()
    C.sq_norm(gb, sq)
    torch.testing.assert_close(sq, (gb.double() ** 2).sum().float().view(1), rtol=1e-4, atol=0)


def test_cross_entropy_forward_backward():
    import pccl

    C = pccl._C
    rows, vocab = 37, 50304
    g = torch.Generator(device=DEV).manual_seed(1)
    logits = (torch.randn(rows, vocab, device=DEV, generator=g) * 3).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device=DEV, generator=g)
    targets[5] = -100
    ref_in = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, targets, reduction="sum", ignore_index=-100)
    ref.backward()
    loss = torch.zeros(1, device=DEV)
    work = logits.clone()
    C.ce_fwd_bwd(work, targets, loss, 0.25, -100)
    torch.testing.assert_close(loss[0], ref.detach(), rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(work.float(), ref_in.grad * 0.25, rtol=2e-2, atol=1e-6)
    assert torch.all(work[5] == 0)
    small = (torch.randn(4, 1000, device=DEV, generator=g)).to(torch.bfloat16)   # vocab not a multiple of 8 vectors
    t2 = torch.randint(0, 1000, (4,), device=DEV, generator=g)
    r2 = small.float().requires_grad_()
    torch.nn.functional.cross_entropy(r2, t2, reduction="sum").backward()
    loss.zero_()
    C.ce_fwd_bwd(small, t2, loss, 1.0, -100)
    torch.testing.assert_close(small.float(), r2.grad, rtol=2e-2, atol=1e-6)


def test_cross_entropy_reports_targets_outside_the_vocabulary():
    """A label that is neither a class nor the ignore index must not be used as an index: its row
    is left out (zero loss, zero gradient) and counted in the error word."""
    import pccl

    C = pccl._C
    rows, vocab = 6, 1024
    g = torch.Generator(device=DEV).manual_seed(3)
    logits = torch.randn(rows, vocab, device=DEV, generator=g).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device=DEV, generator=g)
    targets[1] = -1
    targets[4] = vocab
    good = torch.tensor([0, 2, 3, 5], device=DEV)
    ref_in = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in[good], targets[good], reduction="sum")
    ref.backward()
    loss = torch.zeros(1, device=DEV)
    bad = torch.zeros(1, dtype=torch.int32, device=DEV)
    work = logits.clone()
    C.ce_fwd_bwd(work, targets, loss, 1.0, -100, bad)
    assert int(bad.item()) == 2
    torch.testing.assert_close(loss[0], ref.detach(), rtol=1e-4, atol=1e-3)
    assert torch.all(work[1] == 0) and torch.all(work[4] == 0)
    torch.testing.assert_close(work.float()[good], ref_in.grad[good], rtol=2e-2, atol=1e-6)


def _autograd_reference(cfg, engine, tokens, targets):
    """The same model through torch autograd in fp32 from the engine's master weights."""
    import torch.nn.functional as F

    from pccl.models import gpt

    params = []
    for ui, u in enumerate(engine.units):
        full = engine.master[engine.shard_off[ui]:engine.shard_off[ui + 1]].clone()
        params.append({k: v.clone().requires_grad_() for k, v in gpt.views(u, full).items()})
    B, S = tokens.shape
    p0 = params[0]
    x = F.embedding(tokens, p0["wte"]) + p0["wpe"][:S]
    for p in params[1:]:
        h = F.layer_norm(x, (cfg.d_model,), p["ln1_w"], p["ln1_b"], cfg.ln_eps)
        qkv = F.linear(h, p["qkv_w"], p["qkv_b"]).view(B, S, 3, cfg.n_head, cfg.head_dim)
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, cfg.d_model)
        x = x + F.linear(a, p["proj_w"], p["proj_b"])
        h = F.layer_norm(x, (cfg.d_model,), p["ln2_w"], p["ln2_b"], cfg.ln_eps)
        x = x + F.linear(F.gelu(F.linear(h, p["fc1_w"], p["fc1_b"]), approximate="tanh"), p["fc2_w"], p["fc2_b"])
    x = F.layer_norm(x, (cfg.d_model,), p0["lnf_w"], p0["lnf_b"], cfg.ln_eps)
    logits = F.linear(x, p0["wte"])
    loss = F.cross_entropy(logits.view(B * S, -1), targets.reshape(-1))
    loss.backward()
    return loss.detach(), params


def test_engine_step_matches_autograd():
    """Loss and every parameter gradient of the hand-written forward/backward (bf16) against
    torch autograd in fp32, at world size 1, through the patched backend."""
    import pccl
    from pccl.models import gpt
    from pccl.models.gpt import PRESETS
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine
    from pccl.patch_deepspeed import patch_deepspeed, unpatch_deepspeed
    from pccl.utils.env import init_distributed

    init_distributed()
    comm = pccl.init(heap_bytes=256 << 20, staging_bytes=32 << 20)
    patch_deepspeed(1)
    try:
        cfg = PRESETS["gpt-tiny"]
        engine = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=0.0, weight_decay=0.0), comm=comm, native_gemm=True)
        assert engine.symmetric and engine.local_only
        g = torch.Generator().manual_seed(3)
        toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=g).to(DEV)
        tokens, targets = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
        ref_loss, ref_params = _autograd_reference(cfg, engine, tokens, targets)
        loss = engine.train_step(tokens, targets)
        comm.check()
        torch.testing.assert_close(loss[0], ref_loss, rtol=2e-2, atol=2e-2)
        for ui, u in enumerate(engine.units):
            got = gpt.views(u, engine.grad_shard[engine.shard_off[ui]:engine.shard_off[ui + 1]])
            for name, ref in ref_params[ui].items():
                gr, rf = got[name].float(), ref.grad
                err = (gr - rf).norm() / (rf.norm() + 1e-12)
                assert err < 6e-2, f"unit {u.name} grad {name}: relative error {float(err):.3e}"
        assert engine.launches > 0
        # training moves the loss
        engine2 = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), comm=comm, native_gemm=True)
        losses = [float(engine2.train_step(tokens, targets)) for _ in range(5)]
        assert losses[-1] < losses[0]
        # pinned-host inputs take the same path
        host = toks.cpu().pin_memory()
        l_host = engine.train_step(host[:, :-1], host[:, 1:])
        torch.testing.assert_close(l_host, loss, rtol=1e-3, atol=1e-3)
    finally:
        unpatch_deepspeed()


def test_engine_same_loss_over_torch_backend():
    """The unpatched backend (torch.distributed) drives the same engine to the same loss."""
    import pccl
    from pccl.models.gpt import PRESETS
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine
    from pccl.patch_deepspeed import patch_deepspeed, unpatch_deepspeed
    from pccl.utils.env import init_distributed

    init_distributed()
    cfg = PRESETS["gpt-tiny"]
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=g).to(DEV)
    base = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3))
    assert not base.symmetric
    l_base = [float(base.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(3)]
    comm = pccl.init(heap_bytes=256 << 20, staging_bytes=32 << 20)
    patch_deepspeed(1)
    try:
        ours = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=1e-3), comm=comm, native_gemm=True)
        l_ours = [float(ours.train_step(toks[:, :-1], toks[:, 1:])) for _ in range(3)]
    finally:
        unpatch_deepspeed()
    for a, b in zip(l_base, l_ours):
        assert abs(a - b) < 2e-2, (l_base, l_ours)


@pytest.mark.parametrize("shape", [(8192, 2048), (1000, 6144), (37, 8), (4096, 16384), (5, 72)])
def test_col_sum_matches_fp32_reference(shape):
    import pccl

    T, N = shape
    g = torch.Generator(device=DEV).manual_seed(T + N)
    x = torch.randn(T, N, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.empty(N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):                                  # twice: the tile counters must come back to zero
        out.zero_()
        pccl._C.col_sum(x, out)
        ref = x.float().sum(0)
        torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2 * float(ref.abs().max()))


@pytest.mark.parametrize("shape", [(8192, 2048), (333, 1024), (4096, 4096), (1, 2048), (1237, 2048)])
def test_layer_norm_backward_matches_fp32_reference(shape):
    import pccl

    T, d = shape
    g = torch.Generator(device=DEV).manual_seed(T + d)
    x = (torch.randn(T, d, device=DEV, generator=g) * 2 + 0.5).to(torch.bfloat16)
    dy = torch.randn(T, d, device=DEV, generator=g).to(torch.bfloat16)
    gamma = (torch.randn(d, device=DEV, generator=g) * 0.2 + 1).to(torch.bfloat16)
    beta = torch.zeros(d, device=DEV, dtype=torch.bfloat16)
    _y, mean, rstd = torch.ops.aten.native_layer_norm(x, [d], gamma, beta, 1e-5)
    xr = x.float().requires_grad_()
    gr = gamma.float().requires_grad_()
    br = beta.float().requires_grad_()
    torch.nn.functional.layer_norm(xr, (d,), gr, br, 1e-5).backward(dy.float())
    dg = torch.empty(d, device=DEV, dtype=torch.bfloat16)
    db = torch.empty(d, device=DEV, dtype=torch.bfloat16)
    dx = pccl._C.ln_bwd(dy, x, mean.view(-1), rstd.view(-1), gamma, dg, db)
    assert float((dx.float() - xr.grad).norm() / xr.grad.norm()) < 1e-2
    torch.testing.assert_close(dg.float(), gr.grad, rtol=2e-2, atol=2e-2 * float(gr.grad.abs().max()))
    torch.testing.assert_close(db.float(), br.grad, rtol=2e-2, atol=2e-2 * float(br.grad.abs().max()))
    # with the gradient that flows around the norm added in the same pass
    resid = torch.randn(T, d, device=DEV, generator=g).to(torch.bfloat16)
    dxs = torch.empty(d, device=DEV, dtype=torch.bfloat16)
    dx2 = pccl._C.ln_bwd(dy, x, mean.view(-1), rstd.view(-1), gamma, dg, db, resid, dxs)
    want = xr.grad + resid.float()
    assert float((dx2.float() - want).norm() / want.norm()) < 1e-2
    torch.testing.assert_close(dg.float(), gr.grad, rtol=2e-2, atol=2e-2 * float(gr.grad.abs().max()))
    torch.testing.assert_close(db.float(), br.grad, rtol=2e-2, atol=2e-2 * float(br.grad.abs().max()))
    # ... and the column sums of dx
    sums = dx2.float().sum(0)
    torch.testing.assert_close(dxs.float(), sums, rtol=1e-2, atol=1e-2 * float(sums.abs().max()) + 1e-3)


@pytest.mark.parametrize("shape", [(8192, 2048), (1000, 1024), (37, 8), (5, 24)])
def test_concatenate_three_with_column_sums(shape):
    import pccl

    T, w = shape
    g = torch.Generator(device=DEV).manual_seed(T + 5 * w)
    parts = [torch.randn(T, w, device=DEV, generator=g).to(torch.bfloat16) for _ in range(3)]
    gb = torch.empty(3 * w, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        gb.zero_()
        cat = pccl._C.cat3_col_sum(parts[0], parts[1], parts[2], gb)
        ref = torch.cat(parts, dim=1)
        assert torch.equal(cat, ref)
        sums = ref.float().sum(0)
        torch.testing.assert_close(gb.float(), sums, rtol=1e-2, atol=1e-2 * float(sums.abs().max()) + 1e-3)


@pytest.mark.parametrize("with_branch", [False, True])
@pytest.mark.parametrize("shape", [(8192, 2048), (333, 1024), (2048, 4096), (1, 2048)])
def test_layer_norm_forward_matches_fp32_reference(shape, with_branch):
    import pccl

    T, d = shape
    g = torch.Generator(device=DEV).manual_seed(7 * T + d)
    x = (torch.randn(T, d, device=DEV, generator=g) * 2 + 0.5).to(torch.bfloat16)
    branch = torch.randn(T, d, device=DEV, generator=g).to(torch.bfloat16) if with_branch else None
    gamma = (torch.randn(d, device=DEV, generator=g) * 0.2 + 1).to(torch.bfloat16)
    beta = (torch.randn(d, device=DEV, generator=g) * 0.1).to(torch.bfloat16)
    xs = (x.float() + branch.float()).to(torch.bfloat16) if with_branch else x      # the sum as bf16 stores it
    ref = torch.nn.functional.layer_norm(xs.float(), (d,), gamma.float(), beta.float(), 1e-5)
    mu = xs.float().mean(1)
    rs = (xs.float().var(1, unbiased=False) + 1e-5).rsqrt()
    y, mean, rstd = pccl._C.ln_fwd(x, branch, gamma, beta, 1e-5)
    if with_branch:
        assert torch.equal(branch, xs), "the residual sum must land in the branch buffer, rounded once"
    assert float((y.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert float((y.float() - ref).norm() / ref.norm()) < 4e-3
    torch.testing.assert_close(mean, mu, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(rstd, rs, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("shape", [(4096, 8192), (1000, 4096), (37, 8), (5, 72)])
def test_gelu_forward_and_backward_with_bias_gradient(shape):
    import pccl

    T, N = shape
    g = torch.Generator(device=DEV).manual_seed(T * 3 + N)
    u = (torch.randn(T, N, device=DEV, generator=g) * 2).to(torch.bfloat16)
    u[0, :8] = torch.tensor([-30., -8., -3., -0.5, 0., 0.5, 8., 30.], device=DEV).to(torch.bfloat16)   # tails and zero
    dg = torch.randn(T, N, device=DEV, generator=g).to(torch.bfloat16)
    ur = u.float().requires_grad_()
    ref = torch.nn.functional.gelu(ur, approximate="tanh")
    ref.backward(dg.float())
    y = pccl._C.gelu(u)
    assert torch.isfinite(y.float()).all()
    assert float((y.float() - ref.detach()).abs().max()) <= 1e-2 * float(ref.abs().max()) + 1e-3
    assert float((y.float() - ref.detach()).norm() / ref.norm()) < 4e-3
    gb = torch.empty(N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):                                  # twice: the tile counters must come back to zero
        gb.zero_()
        du = pccl._C.gelu_bwd_col_sum(dg, u, gb)
        assert torch.isfinite(du.float()).all()
        assert float((du.float() - ur.grad).norm() / ur.grad.norm()) < 4e-3
        want = du.float().sum(0)
        torch.testing.assert_close(gb.float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()) + 1e-3)


@pytest.mark.parametrize("fused_gelu_gemm,overlap_wgrad,gelu_bwd_gemm",
                         [(False, False, False), (True, False, False), (False, True, False), (False, False, True)])
def test_engine_fused_kernels_match_autograd_at_width_1024(fused_gelu_gemm, overlap_wgrad, gelu_bwd_gemm):
    """A two-block model wide enough (d = 1024) for the fused add+layer-norm, layer-norm backward
    with residual, GELU and GELU-backward kernels, with FC1 optionally on the tcgen05 GEMM whose
    epilogue applies the GELU: loss and every gradient against torch autograd in fp32."""
    from pccl.models import gpt
    from pccl.models.gpt import GPTConfig
    from pccl.parallel.backend import TorchBackend
    from pccl.parallel.zero3 import OptimConfig, Zero3Engine
    from pccl.utils.env import init_distributed

    init_distributed()
    cfg = GPTConfig(2, 1024, 8, 4096, vocab=2048, seq_len=128, name="gpt-test-1024")
    engine = Zero3Engine(cfg, TorchBackend(), OptimConfig(lr=0.0, weight_decay=0.0), fused_gelu_gemm=fused_gelu_gemm,
                         overlap_wgrad=overlap_wgrad, fused_gelu_bwd_gemm=gelu_bwd_gemm, native_gemm=True)
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=g).to(DEV)
    tokens, targets = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    ref_loss, ref_params = _autograd_reference(cfg, engine, tokens, targets)
    before = gpt.native_launches
    loss = engine.train_step(tokens, targets)
    if overlap_wgrad:
        for _ in range(3):                              # repeated steps reuse the gradient buffers across streams
            loss = engine.train_step(tokens, targets)
    # per block: 2 ln_fwd, GELU (its own kernel, or none when it rides in FC1's epilogue), gelu_bwd, cat3,
    # 2 x (ln_bwd + finalize), and the twelve dense products (4 forward, 4 data gradients, 4 weight
    # gradients); head: ln_fwd, ln_bwd + finalize and its three dense products
    # (with gelu_bwd_gemm the GELU backward rides in the data-gradient GEMM of FC2 and leaves a column sum
    # behind: same count)
    per_block = 8 + (0 if fused_gelu_gemm else 1) + 12
    expected = cfg.n_layer * per_block + 3 + 3
    if overlap_wgrad:
        before = gpt.native_launches - expected
    engine.check_errors()
    assert gpt.native_launches - before == expected
    torch.testing.assert_close(loss[0], ref_loss, rtol=2e-2, atol=2e-2)
    for ui, u in enumerate(engine.units):
        got = gpt.views(u, engine.grad_shard[engine.shard_off[ui]:engine.shard_off[ui + 1]])
        for name, ref in ref_params[ui].items():
            gr, rf = got[name].float(), ref.grad
            err = (gr - rf).norm() / (rf.norm() + 1e-12)
            assert err < 6e-2, f"unit {u.name} grad {name}: relative error {float(err):.3e}"
