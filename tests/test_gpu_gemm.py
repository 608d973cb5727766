"""tcgen05 GEMM and fused all-gather+GEMM against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


def check_close(y, ref, K):
    # bf16 inputs, fp32 accumulation, one rounding to bf16 at the end
    err = (y.float() - ref).abs().max()
    tol = 2e-2 * ref.abs().max() + 1e-3
    assert float(err) <= float(tol), f"max abs err {float(err):.4g} > {float(tol):.4g}"
    rel = (y.float() - ref).norm() / ref.norm()
    assert float(rel) < 5e-3, f"relative error {float(rel):.3e}"


@pytest.mark.parametrize("two_cta", [False, True], ids=["one_sm", "cta_pair"])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 128), (384, 768, 2048), (1000, 520, 328), (8192, 6144, 2048)])
def test_gemm_matches_fp32_reference(shape, two_cta):
    import pccl

    M, N, K = shape
    A, W = rnd((M, K), 1), rnd((N, K), 2, 0.05)
    bias = rnd((N,), 3)
    y, err = pccl._C.gemm(A, W, bias, None, two_cta)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = A.float() @ W.float().t() + bias.float()
    check_close(y, ref, K)
    y2, err2 = pccl._C.gemm(A, W, None, None, two_cta)
    torch.cuda.synchronize()
    assert int(err2.item()) == 0
    check_close(y2, A.float() @ W.float().t(), K)


@pytest.mark.parametrize("two_cta", [False, True], ids=["one_sm", "cta_pair"])
@pytest.mark.parametrize("shape", [(256, 512, 128), (1000, 520, 328), (2048, 4096, 1024)])
def test_gemm_with_gelu_epilogue(shape, two_cta):
    """One kernel, two outputs: the pre-activation (kept for the backward pass) and its GELU."""
    import pccl

    M, N, K = shape
    A, W = rnd((M, K), 1), rnd((N, K), 2, 0.08)
    bias = rnd((N,), 3)
    u, g, err = pccl._C.gemm_gelu(A, W, bias, two_cta)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref_u = A.float() @ W.float().t() + bias.float()
    check_close(u, ref_u, K)
    y_plain, _ = pccl._C.gemm(A, W, bias, None, two_cta)
    assert torch.equal(u, y_plain), "the pre-activation must not depend on the second output"
    ref_g = torch.nn.functional.gelu(u.float(), approximate="tanh")      # the activation reads the stored bf16 value
    assert float((g.float() - ref_g).abs().max()) <= 1e-2 * float(ref_g.abs().max()) + 1e-3
    assert float((g.float() - ref_g).norm() / ref_g.norm()) < 4e-3


def test_linear_wrapper_and_identity():
    from pccl.ops.gemm import linear

    K = 256
    x = rnd((3, 50, K), 5)
    eye = torch.eye(K, device=DEV, dtype=torch.bfloat16)
    y = linear(x, eye, check=True)
    assert torch.equal(y, x)                     # exact: one non-zero product per output
    w = rnd((512, K), 6, 0.1)
    y = linear(x, w, check=True)
    check_close(y.view(-1, 512), x.view(-1, K).float() @ w.float().t(), K)
    with pytest.raises(RuntimeError):
        linear(rnd((4, 12), 1), rnd((8, 12), 2))   # K not a multiple of 8
    # one-CTA form through the wrapper, and the two-output form
    y1 = linear(x, w, check=True, two_cta=False)
    check_close(y1.view(-1, 512), x.view(-1, K).float() @ w.float().t(), K)
    from pccl.ops.gemm import linear_gelu

    b = rnd((512,), 7)
    u, g = linear_gelu(x, w, b, check=True)
    assert u.shape == (3, 50, 512) and g.shape == u.shape
    check_close(u.view(-1, 512), x.view(-1, K).float() @ w.float().t() + b.float(), K)
    ref_g = torch.nn.functional.gelu(u.float(), approximate="tanh")
    assert float((g.float() - ref_g).abs().max()) <= 1e-2 * float(ref_g.abs().max()) + 1e-3


@pytest.mark.parametrize("two_cta", [False, True], ids=["one_sm", "cta_pair"])
@pytest.mark.parametrize("P,me", [(2, 0), (4, 3), (8, 5)])
def test_fused_gather_gemm_with_local_peers(P, me, two_cta):
    """The fused kernel with peers that are local buffers: gatherer CTAs pull every shard
    into the local weight buffer while the GEMM CTAs multiply panel by panel."""
    import pccl

    M, K = 512, 512
    N = P * 256 * 2
    A = rnd((M, K), 11)
    shards = [rnd((N // P, K), 20 + p, 0.05) for p in range(P)]
    bias = rnd((N,), 40)
    w_full = torch.zeros((N, K), device=DEV, dtype=torch.bfloat16)
    y, err = pccl._C.ag_gemm_local(A, shards, me, w_full, bias, 4, two_cta)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    W = torch.cat(shards)
    assert torch.equal(w_full, W), "the gathered weight must be a bit-exact copy of the shards"
    check_close(y, A.float() @ W.float().t() + bias.float(), K)


@pytest.mark.parametrize("P,me,ppc", [(2, 1, 0), (4, 0, 1), (8, 6, 0)])
def test_fused_gather_gemm_fed_by_the_copy_engines(P, me, ppc):
    """The other way to feed the fused kernel: no gatherer CTAs; copies on a second stream bring
    the panels, stream-ordered 32-bit writes raise their flags, every CTA multiplies."""
    import pccl

    M, K = 768, 1024
    N = P * 256 * 2
    A = rnd((M, K), 12)
    shards = [rnd((N // P, K), 60 + p, 0.05) for p in range(P)]
    bias = rnd((N,), 41)
    w_full = torch.zeros((N, K), device=DEV, dtype=torch.bfloat16)
    for _ in range(2):                      # twice: the copy stream and its events are reused
        y, err = pccl._C.ag_gemm_local(A, shards, me, w_full, bias, 0, True, True, ppc)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        W = torch.cat(shards)
        assert torch.equal(w_full, W)
        check_close(y, A.float() @ W.float().t() + bias.float(), K)
        w_full.zero_()


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 256), (960, 512, 328), (4096, 2048, 8192),
                                   (8192, 8192, 2048)])
def test_gemm_data_gradient_layout(shape):
    """dx = dy @ W with W stored [K_contract, N]: the second operand is read 'transposed in memory'."""
    import pccl

    M, N, K = shape
    dy, W = rnd((M, K), 1), rnd((K, N), 2, 0.05)
    y = pccl._C.gemm_ex(dy, W, False, True)
    torch.cuda.synchronize()
    assert int(pccl._C.gemm_error_word(0).item()) == 0
    check_close(y, dy.float() @ W.float(), K)


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 256), (2048, 2048, 8192), (6144, 2048, 8192), (50304, 1024, 4096),
                                   (320, 192, 1000)])
def test_gemm_weight_gradient_layout(shape):
    """dW = dy^T @ x with both operands stored [tokens, features]: both are read 'transposed in
    memory', including a token count that is not a multiple of the 64-wide k block and an output
    that is not a multiple of the 256-wide tile."""
    import pccl

    M, N, K = shape
    dy, x = rnd((K, M), 1, 0.1), rnd((K, N), 2, 0.1)
    out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    y = pccl._C.gemm_ex(dy, x, True, True, None, out)
    torch.cuda.synchronize()
    assert int(pccl._C.gemm_error_word(0).item()) == 0
    assert y.data_ptr() == out.data_ptr()
    check_close(y, dy.float().t() @ x.float(), K)


def test_gemm_transposed_first_operand_only():
    import pccl

    M, N, K = 384, 512, 320
    a, w = rnd((K, M), 3), rnd((N, K), 4, 0.1)
    bias = rnd((N,), 5)
    y = pccl._C.gemm_ex(a, w, True, False, bias)
    torch.cuda.synchronize()
    check_close(y, a.float().t() @ w.float().t() + bias.float(), K)
    with pytest.raises(RuntimeError):
        pccl._C.gemm_ex(rnd((64, 100), 1), w[:, :64].contiguous(), True, False)     # M = 100 is not a multiple of 64


@pytest.mark.parametrize("shape,layout", [((8192, 2048, 2048), "nt"), ((4096, 2048, 8192), "nn"), ((2048, 2048, 8192), "tn"),
                                          ((512, 512, 8192), "nt"), ((768, 1280, 4096), "tn"), ((8192, 6144, 2048), "nt"),
                                          ((1000, 2048, 3072), "nt")])
def test_last_round_split_along_k(shape, layout):
    """Shapes whose last round of tiles is only partly filled (or that have fewer tiles than CTA
    pairs): the leading tiles are computed by two or more pairs, the partial sums meet in the
    finisher's epilogue.  Same result as the unsplit launch up to fp32 summation order, same as
    the fp32 reference within the usual tolerance; bias and the GELU output ride along."""
    import pccl

    C = pccl._C
    M, N, K = shape
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert C.gemm_sk_tiles(M, N, K, sms) > 0, "pick shapes that are split"
    a, w = rnd((M, K), 1), rnd((N, K), 2, 0.05)
    bias = rnd((N,), 3)
    ref = a.float() @ w.float().t()
    if layout == "nt":
        run = lambda: C.gemm_ex(a, w, False, False, bias, None)  # noqa: E731
        ref = ref + bias.float()
    elif layout == "nn":
        wt = w.t().contiguous()
        run = lambda: C.gemm_ex(a, wt, False, True, None, None)  # noqa: E731
    else:
        at_, wt = a.t().contiguous(), w.t().contiguous()
        run = lambda: C.gemm_ex(at_, wt, True, True, None, None)  # noqa: E731
    try:
        C.gemm_set_wide(0)                       # single tiles: the form that splits
        C.gemm_set_split_last_wave(False)
        y_plain = run()
        C.gemm_set_split_last_wave(True, True)   # shapes with fewer tiles than CTA pairs too
        for _ in range(3):                       # repeated launches reuse the scratch and its flags
            y_split = run()
            torch.cuda.synchronize()
            assert int(C.gemm_error_word(0).item()) == 0
            check_close(y_split, ref, K)
            assert float((y_split.float() - y_plain.float()).abs().max()) <= 1e-2 * float(ref.abs().max()) + 1e-3
        if layout == "nt":
            u, g, err = C.gemm_gelu(a, w, bias, True)
            torch.cuda.synchronize()
            assert int(err.item()) == 0
            assert torch.equal(u, y_split)
            ref_g = torch.nn.functional.gelu(u.float(), approximate="tanh")
            assert float((g.float() - ref_g).abs().max()) <= 1e-2 * float(ref_g.abs().max()) + 1e-3
    finally:
        C.gemm_set_split_last_wave(True)
        C.gemm_set_wide(-1)


@pytest.mark.parametrize("shape", [(512, 768, 256), (960, 512, 328), (8192, 8192, 2048), (1024, 2048, 4096)])
def test_gemm_with_gelu_backward_epilogue(shape):
    """du = (dy @ W) * gelu'(u): the GELU backward as the epilogue of the data-gradient product (W stored
    [K, N], read as it lies), with and without tiles that are split along K."""
    import pccl

    M, N, K = shape
    dy, W = rnd((M, K), 1), rnd((K, N), 2, 0.05)
    u = rnd((M, N), 3, 1.5)
    du = pccl._C.gemm_ex(dy, W, False, True, None, None, u)
    torch.cuda.synchronize()
    assert int(pccl._C.gemm_error_word(0).item()) == 0
    uf = u.float().requires_grad_()
    torch.nn.functional.gelu(uf, approximate="tanh").sum().backward()
    ref = (dy.float() @ W.float()) * uf.grad
    check_close(du, ref, K)


@pytest.mark.parametrize("shape,layout", [((8192, 2048, 2048), "nt"), ((1000, 520, 328), "nt"), ((4096, 2048, 8192), "nn"),
                                          ((2048, 2048, 4096), "tn"), ((256, 256, 64), "nt"), ((8192, 6144, 2048), "nt")])
def test_tiles_drawn_at_run_time(shape, layout):
    """The other way of dealing out tiles: every CTA pair draws its next tile from a counter that runs on
    from launch to launch.  Repeated launches, with bias, same results as the fixed shares."""
    import pccl

    C = pccl._C
    M, N, K = shape
    a, w = rnd((M, K), 1), rnd((N, K), 2, 0.05)
    bias = rnd((N,), 3)
    ref = a.float() @ w.float().t()
    if layout == "nt":
        run = lambda: C.gemm_ex(a, w, False, False, bias, None)  # noqa: E731
        ref = ref + bias.float()
    elif layout == "nn":
        wt = w.t().contiguous()
        run = lambda: C.gemm_ex(a, wt, False, True, None, None)  # noqa: E731
    else:
        at_, wt = a.t().contiguous(), w.t().contiguous()
        run = lambda: C.gemm_ex(at_, wt, True, True, None, None)  # noqa: E731
    try:
        C.gemm_set_dynamic_tiles(True)
        for _ in range(4):
            y = run()
            torch.cuda.synchronize()
            assert int(C.gemm_error_word(0).item()) == 0
            check_close(y, ref, K)
    finally:
        C.gemm_set_dynamic_tiles(False)


@pytest.mark.parametrize("shape,layout", [((8192, 6144, 2048), "nt"), ((300, 256, 64), "nt"), ((1000, 520, 328), "nt"),
                                          ((12576, 2048, 512), "nt"), ((4096, 2048, 8192), "nn"), ((1280, 512, 320), "tn"),
                                          ((2048, 2048, 8192), "tn")])
@pytest.mark.parametrize("dynamic", [False, True], ids=["dealt_out", "drawn_at_run_time"])
def test_units_of_two_row_tiles_sharing_w(shape, layout, dynamic):
    """The wide form of the CTA-pair kernel: two vertically adjacent 256 x 256 tiles share their W half in
    shared memory and fill both TMEM accumulators.  Same result as the plain form, bit for bit (the same
    products are summed in the same order), for full units, a unit whose lower tile is partly or wholly
    past M, with bias, in all three layouts, with the units dealt out in advance or drawn from the counter."""
    import pccl

    C = pccl._C
    M, N, K = shape
    a, w = rnd((M, K), 1), rnd((N, K), 2, 0.05)
    bias = rnd((N,), 3)
    ref = a.float() @ w.float().t()
    if layout == "nt":
        run = lambda: C.gemm_ex(a, w, False, False, bias, None)  # noqa: E731
        ref = ref + bias.float()
    elif layout == "nn":
        wt = w.t().contiguous()
        run = lambda: C.gemm_ex(a, wt, False, True, None, None)  # noqa: E731
    else:
        at_, wt = a.t().contiguous(), w.t().contiguous()
        run = lambda: C.gemm_ex(at_, wt, True, True, None, None)  # noqa: E731
    C.gemm_set_split_last_wave(False)
    try:
        C.gemm_set_wide(0)
        plain = run()
        C.gemm_set_wide(1)
        C.gemm_set_dynamic_tiles(dynamic)
        for _ in range(3):
            y = run()
            torch.cuda.synchronize()
            assert int(C.gemm_error_word(0).item()) == 0
            check_close(y, ref, K)
            assert torch.equal(y, plain)
    finally:
        C.gemm_set_dynamic_tiles(False)
        C.gemm_set_wide(-1)
        C.gemm_set_split_last_wave(True)
