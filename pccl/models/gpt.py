"""GPT-2-style decoder written as explicit forward and backward functions over flat
parameter views.

The reference ships no model: its DeepSpeed hook (``pccl/patch_deepspeed.py:95-126``)
expects an external GPT training script.  The benchmark configurations name two models
(1.3B: 24 layers, d_model 2048, 16 heads, FFN 8192; 7B: 32 layers, d_model 4096, 32 heads,
FFN 16384; GELU, vocabulary 50304, sequence 2048, tied embeddings, N(0, 0.02) init), and
this module provides them in the form a ZeRO-3 engine wants: parameters grouped in
"units" that are gathered and released one at a time, a forward that keeps only what the
backward needs, and a backward that writes weight gradients straight into a flat
gradient buffer (no autograd graph, no per-parameter ``.grad`` tensors to copy).

Every dense product (the four linear layers of a block forward, their data and weight
gradients, the output projection and its gradients) runs on this library's tcgen05 GEMM
(``pccl/csrc/gemm_sm100.cu``) when ``native_gemm`` is on and the operands qualify; the weight and
data gradients read their operands as they lie in memory (``pccl.ops.gemm.matmul_tn`` /
``matmul_nn``), so nothing is transposed by a copy.  With ``native_gemm`` off, or for operands the
kernel does not take, the same products go to cuBLAS through ``torch`` (the baseline arm).  The
two GEMMs that directly consume a freshly gathered weight (QKV and FC1) can be replaced by the
fused all-gather+GEMM kernel through the ``linear_fwd`` hook.  The attention core uses
``scaled_dot_product_attention`` under a local autograd scope.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class GPTConfig:
    n_layer: int
    d_model: int
    n_head: int
    d_ff: int
    vocab: int = 50304
    seq_len: int = 2048
    init_std: float = 0.02
    ln_eps: float = 1e-5
    name: str = "gpt"

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    def num_params(self) -> int:
        return sum(u.numel for u in unit_specs(self))

    def flops_per_token(self) -> float:
        """Forward+backward matmul FLOPs per token: 6 per dense weight, plus causal
        attention (QK^T and PV, half of the square)."""
        dense = self.n_layer * (4 * self.d_model * self.d_model + 2 * self.d_model * self.d_ff) + self.vocab * self.d_model
        attn = self.n_layer * self.seq_len * self.d_model
        return 6.0 * dense + 6.0 * attn


PRESETS: Dict[str, GPTConfig] = {
    "gpt-1.3b": GPTConfig(24, 2048, 16, 8192, name="gpt-1.3b"),
    "gpt-7b": GPTConfig(32, 4096, 32, 16384, name="gpt-7b"),
    "gpt-350m": GPTConfig(24, 1024, 16, 4096, name="gpt-350m"),
    "gpt-tiny": GPTConfig(2, 256, 4, 1024, vocab=1024, seq_len=128, name="gpt-tiny"),
}


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    init: str           # "normal" | "zeros" | "ones"
    offset: int = 0     # element offset inside the unit

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


@dataclass
class UnitSpec:
    name: str
    params: List[ParamSpec]
    numel: int = 0      # unpadded size; parameters are laid out back to back, 256-element aligned


_ALIGN = 256


def _layout(name: str, params: List[ParamSpec]) -> UnitSpec:
    off = 0
    for p in params:
        off = (off + _ALIGN - 1) // _ALIGN * _ALIGN
        p.offset = off
        off += p.numel
    return UnitSpec(name, params, off)


def unit_specs(cfg: GPTConfig) -> List[UnitSpec]:
    """Unit 0 holds the embeddings and the final layer norm (the head needs both and the
    token embedding is tied to the output projection); units 1..L are the blocks."""
    d, f = cfg.d_model, cfg.d_ff
    units = [_layout("embed", [
        ParamSpec("wte", (cfg.vocab, d), "normal"),
        ParamSpec("wpe", (cfg.seq_len, d), "normal"),
        ParamSpec("lnf_w", (d,), "ones"),
        ParamSpec("lnf_b", (d,), "zeros"),
    ])]
    for i in range(cfg.n_layer):
        units.append(_layout(f"layer{i}", [
            ParamSpec("qkv_w", (3 * d, d), "normal"),
            ParamSpec("fc1_w", (f, d), "normal"),
            ParamSpec("proj_w", (d, d), "normal"),
            ParamSpec("fc2_w", (d, f), "normal"),
            ParamSpec("qkv_b", (3 * d,), "zeros"),
            ParamSpec("fc1_b", (f,), "zeros"),
            ParamSpec("proj_b", (d,), "zeros"),
            ParamSpec("fc2_b", (d,), "zeros"),
            ParamSpec("ln1_w", (d,), "ones"),
            ParamSpec("ln1_b", (d,), "zeros"),
            ParamSpec("ln2_w", (d,), "ones"),
            ParamSpec("ln2_b", (d,), "zeros"),
        ]))
    return units


def views(unit: UnitSpec, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Named parameter views into a flat buffer that holds the unit."""
    return {p.name: flat[p.offset:p.offset + p.numel].view(p.shape) for p in unit.params}


def init_unit(unit: UnitSpec, flat: torch.Tensor, cfg: GPTConfig, seed: int) -> None:
    """Fill a full (gathered-size) fp32 buffer with the unit's initial values.  The values
    depend on (seed, unit, parameter) only, never on how many ranks shard the unit."""
    flat.zero_()
    for idx, p in enumerate(unit.params):
        v = flat[p.offset:p.offset + p.numel]
        if p.init == "normal":
            g = torch.Generator(device=flat.device).manual_seed(seed * 1000003 + idx)
            v.normal_(0.0, cfg.init_std, generator=g)
        elif p.init == "ones":
            v.fill_(1.0)


# ---------------------------------------------------------------------------- layer math
LinearFwd = Callable[[torch.Tensor, torch.Tensor, Optional[torch.Tensor], str], torch.Tensor]


def _default_linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], which: str) -> torch.Tensor:
    return mm_nt(x, w, b)


def _gemm_ok(*ts: torch.Tensor) -> bool:
    return native_gemm and bool(_kernels()) and all(
        t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.is_contiguous() and t.data_ptr() % 16 == 0 for t in ts)


def mm_nt(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T (+ b)."""
    if _gemm_ok(x, w) and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 and (b is None or b.is_contiguous()):
        global native_launches
        native_launches += 1
        return _kernels().gemm_ex(x, w, False, False, b, None)
    return F.linear(x, w, b)


def mm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a[M,K] @ b[K,N]: the data gradient of a linear layer whose weight is stored [out, in]."""
    if _gemm_ok(a, b) and (out is None or _gemm_ok(out)) and b.shape[1] % 64 == 0 and b.shape[0] % 8 == 0:
        global native_launches
        native_launches += 1
        return _kernels().gemm_ex(a, b, False, True, None, out)
    return torch.mm(a, b, out=out) if out is not None else torch.mm(a, b)


def mm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a[K,M]^T @ b[K,N]: the weight gradient of a linear layer, operands stored [tokens, features]."""
    if _gemm_ok(a, b) and (out is None or _gemm_ok(out)) and a.shape[1] % 64 == 0 and b.shape[1] % 64 == 0 \
            and a.shape[0] % 8 == 0:
        global native_launches
        native_launches += 1
        return _kernels().gemm_ex(a, b, True, True, None, out)
    return torch.mm(a.t(), b, out=out) if out is not None else torch.mm(a.t(), b)


def _ln_fwd(x, w, b, eps, branch=None):
    """Layer norm of ``x`` (+ ``branch``).  With ``branch`` the sum is formed in the same pass,
    written over ``branch`` and returned as the new residual stream: (y, mean, rstd, x_sum)."""
    if _fast(x) and x.shape[-1] in (1024, 2048, 4096) and w.is_contiguous() and b.is_contiguous() \
            and (branch is None or _fast(branch)):
        global native_launches
        native_launches += 1
        y, mean, rstd = _kernels().ln_fwd(x, branch, w, b, eps)
        return y, mean, rstd, (x if branch is None else branch)
    if branch is not None:
        x = branch.add_(x)
    y, mean, rstd = torch.ops.aten.native_layer_norm(x, [x.shape[-1]], w, b, eps)
    return y, mean, rstd, x


_native = None
native_launches = 0     # kernels of this library launched by the functions below
native_gemm = True       # dense products on the library's tcgen05 GEMM (off: cuBLAS through torch; set by the engine)
fused_gelu_gemm = False  # FC1 on the tcgen05 GEMM with the GELU in its epilogue (set by the engine)
fused_gelu_bwd_gemm = False  # the GELU backward as the epilogue of the data-gradient GEMM in front of it (with native_gemm)


def _kernels():
    """The native extension, or False where it cannot be loaded (pure-PyTorch fallback)."""
    global _native
    if _native is None:
        try:
            from .. import build_kernels

            _native = build_kernels.load()
        except Exception:  # noqa: BLE001
            _native = False
    return _native


def _fast(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.is_contiguous() and bool(_kernels())


def _ln_bwd(dy, x, mean, rstd, w, b, gw, gb, resid=None, dx_sum=None):
    """dx of a layer norm (+ ``resid``, the gradient flowing around it); writes gw, gb and, into
    ``dx_sum`` when given, the column sums of dx (the bias gradient of the linear layer that
    produced the normalised tensor's input)."""
    if _fast(dy) and _fast(x) and x.shape[-1] in (1024, 2048, 4096) and gw.is_contiguous() and gb.is_contiguous() \
            and (resid is None or _fast(resid)) and (dx_sum is None or dx_sum.is_contiguous()):
        # one pass over dy and x: dx plus the weight/bias gradients, written in place
        global native_launches
        native_launches += 2
        return _kernels().ln_bwd(dy, x, mean.view(-1), rstd.view(-1), w, gw, gb, resid, dx_sum)
    dx, dw, db = torch.ops.aten.native_layer_norm_backward(dy, x, [x.shape[-1]], mean.view(-1, 1), rstd.view(-1, 1), w, b,
                                                           [True, True, True])
    gw.copy_(dw)
    gb.copy_(db)
    if resid is not None:
        dx = dx.add_(resid)
    if dx_sum is not None:
        torch.sum(dx, dim=0, out=dx_sum)
    return dx


def _bias_grad(dy: torch.Tensor, gb: torch.Tensor) -> None:
    """gb = column sums of dy."""
    if _fast(dy) and dy.shape[1] % 8 == 0 and gb.is_contiguous():
        global native_launches
        native_launches += 1
        _kernels().col_sum(dy, gb)
    else:
        torch.sum(dy, dim=0, out=gb)


def _fc1_gelu(h: torch.Tensor, p: Dict[str, torch.Tensor], linear_fwd: LinearFwd):
    """u = h @ fc1_w^T + fc1_b and g = gelu(u)."""
    global native_launches
    w, b = p["fc1_w"], p["fc1_b"]
    if fused_gelu_gemm and linear_fwd is _default_linear and _fast(h) and _fast(w) and b.is_contiguous() \
            and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
        native_launches += 1
        u, g, _err = _kernels().gemm_gelu(h, w, b)
        return u, g
    u = linear_fwd(h, w, b, "fc1")
    if _fast(u) and u.numel() % 8 == 0:
        native_launches += 1
        return u, _kernels().gelu(u)
    return u, F.gelu(u, approximate="tanh")


def _gelu_bwd(dg: torch.Tensor, u: torch.Tensor, gb: torch.Tensor) -> torch.Tensor:
    """du = dg * gelu'(u); the bias gradient of the layer in front (column sums of du) goes to gb."""
    if _fast(dg) and _fast(u) and u.shape[1] % 8 == 0 and gb.is_contiguous():
        global native_launches
        native_launches += 1
        return _kernels().gelu_bwd_col_sum(dg, u, gb)
    du = torch.ops.aten.gelu_backward(dg, u, approximate="tanh")
    torch.sum(du, dim=0, out=gb)
    return du


def layer_forward_deferred(x: torch.Tensor, branch: Optional[torch.Tensor], p: Dict[str, torch.Tensor], cfg: GPTConfig,
                           batch: int, linear_fwd: LinearFwd = _default_linear):
    """One transformer block whose residual adds ride on the layer norms.

    The block's input is ``x + branch`` (``branch``: the previous block's MLP output, not yet
    added; None for the first block).  Returns ``(x2, mlp_out, ctx)``: the block's output is
    ``x2 + mlp_out``, left unsummed so the next layer norm adds it in its own pass."""
    T, d = x.shape
    S, H, dh = T // batch, cfg.n_head, cfg.head_dim
    h1, mean1, rstd1, x = _ln_fwd(x, p["ln1_w"], p["ln1_b"], cfg.ln_eps, branch)
    qkv = linear_fwd(h1, p["qkv_w"], p["qkv_b"], "qkv")                  # [T, 3d]
    q, k, v = (t.transpose(1, 2) for t in qkv.view(batch, S, 3, H, dh).unbind(2))   # [B, H, S, dh] views
    qd, kd, vd = (t.detach().requires_grad_() for t in (q, k, v))
    with torch.enable_grad():
        att = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True)            # [B, H, S, dh]
    a = att.detach().transpose(1, 2).reshape(T, d)
    o = mm_nt(a, p["proj_w"], p["proj_b"])
    h2, mean2, rstd2, x2 = _ln_fwd(x, p["ln2_w"], p["ln2_b"], cfg.ln_eps, o)       # x2 = x + o, in o's memory
    u, g = _fc1_gelu(h2, p, linear_fwd)                                  # [T, f]
    m = mm_nt(g, p["fc2_w"], p["fc2_b"])
    ctx = (x, mean1, rstd1, h1, qd, kd, vd, att, a, x2, mean2, rstd2, h2, u, g)
    return x2, m, ctx


def layer_forward(x: torch.Tensor, p: Dict[str, torch.Tensor], cfg: GPTConfig, batch: int,
                  linear_fwd: LinearFwd = _default_linear):
    """x: [T, d] with T = batch * seq.  Returns (y, ctx)."""
    x2, m, ctx = layer_forward_deferred(x, None, p, cfg, batch, linear_fwd)
    return m.add_(x2), ctx


def _cat_qkv_grads(dq, dk, dv, T: int, d: int, gb: torch.Tensor) -> torch.Tensor:
    """[T, 3d] gradient of the packed QKV projection and its column sums (the QKV bias gradient).
    The attention backward returns its gradients in the memory order of q, k, v ([B, S, H, dh]
    underneath), so their [T, d] forms are views."""
    parts = [t.transpose(1, 2).reshape(T, d) for t in (dq, dk, dv)]
    if all(_fast(t) for t in parts) and d % 8 == 0 and gb.is_contiguous():
        global native_launches
        native_launches += 1
        return _kernels().cat3_col_sum(parts[0], parts[1], parts[2], gb)
    dqkv = torch.cat(parts, dim=1)
    torch.sum(dqkv, dim=0, out=gb)
    return dqkv


def layer_backward(dy: torch.Tensor, ctx, p: Dict[str, torch.Tensor], gr: Dict[str, torch.Tensor], cfg: GPTConfig,
                   batch: int, dy_sum: Optional[torch.Tensor] = None, dx_sum: Optional[torch.Tensor] = None,
                   side: Optional["torch.cuda.Stream"] = None) -> torch.Tensor:
    """Returns dx; writes every parameter gradient of the layer into the views ``gr``.

    ``dy_sum``: the column sums of ``dy`` when the kernel that produced ``dy`` already formed them
    (they are this block's FC2 bias gradient).  ``dx_sum``: a [d] tensor that receives the column
    sums of the returned dx, for the block below.  ``side``: a second stream for the four
    weight-gradient GEMMs, which nothing in the block's own backward chain depends on; they then
    run beside the memory-bound kernels of the chain (GELU backward, layer-norm backward, the
    q/k/v packing) instead of between them.  The current stream waits for ``side`` before the
    function returns, and every tensor a side-stream GEMM reads stays referenced until then."""
    global native_launches
    x, mean1, rstd1, h1, qd, kd, vd, att, a, x2, mean2, rstd2, h2, u, g = ctx
    T, d = x.shape
    S, H, dh = T // batch, cfg.n_head, cfg.head_dim
    main = torch.cuda.current_stream(dy.device) if side is not None else None

    def wgrad(dy_, x_, gw):
        if side is None:
            mm_tn(dy_, x_, out=gw)
            return
        side.wait_stream(main)                  # dy_ and x_ are complete, gw's previous reader is done
        with torch.cuda.stream(side):
            mm_tn(dy_, x_, out=gw)

    if dy_sum is not None:
        gr["fc2_b"].copy_(dy_sum)
    else:
        _bias_grad(dy, gr["fc2_b"])
    wgrad(dy, g, gr["fc2_w"])
    if fused_gelu_bwd_gemm and _gemm_ok(dy, p["fc2_w"], u) and u.shape[1] % 64 == 0 and dy.shape[1] % 8 == 0:
        # du = (dy @ fc2_w) * gelu'(u) in one kernel: the product never exists in memory; the bias
        # gradient of FC1 is the column sum of du
        native_launches += 1
        du = _kernels().gemm_ex(dy, p["fc2_w"], False, True, None, None, u)
        _bias_grad(du, gr["fc1_b"])
    else:
        dg = mm_nn(dy, p["fc2_w"])
        du = _gelu_bwd(dg, u, gr["fc1_b"])
    wgrad(du, h2, gr["fc1_w"])
    dh2 = mm_nn(du, p["fc1_w"])
    # dx2 is the gradient of the attention projection's output: its column sums are proj_b's gradient
    dx2 = _ln_bwd(dh2, x2, mean2, rstd2, p["ln2_w"], p["ln2_b"], gr["ln2_w"], gr["ln2_b"], resid=dy, dx_sum=gr["proj_b"])
    wgrad(dx2, a, gr["proj_w"])
    da = mm_nn(dx2, p["proj_w"])
    datt = da.view(batch, S, H, dh).transpose(1, 2)
    dq, dk, dv = torch.autograd.grad(att, (qd, kd, vd), datt)
    dqkv = _cat_qkv_grads(dq, dk, dv, T, d, gr["qkv_b"])
    wgrad(dqkv, h1, gr["qkv_w"])
    dh1 = mm_nn(dqkv, p["qkv_w"])
    dx = _ln_bwd(dh1, x, mean1, rstd1, p["ln1_w"], p["ln1_b"], gr["ln1_w"], gr["ln1_b"], resid=dx2, dx_sum=dx_sum)
    if side is not None:
        main.wait_stream(side)                  # the gradient buffer is complete for whoever reads it next
    return dx


def embed_forward(tokens: torch.Tensor, p: Dict[str, torch.Tensor]) -> torch.Tensor:
    """tokens: [B, S] int64 -> [B*S, d]."""
    B, S = tokens.shape
    x = F.embedding(tokens, p["wte"])
    x = x + p["wpe"][:S].unsqueeze(0)
    return x.view(B * S, -1)


def embed_backward(dx: torch.Tensor, tokens: torch.Tensor, gr: Dict[str, torch.Tensor]) -> None:
    """Accumulates into gr["wte"] (the head already wrote its share) and writes gr["wpe"]."""
    B, S = tokens.shape
    gr["wte"].index_add_(0, tokens.reshape(-1), dx)
    gw = gr["wpe"]
    gw.zero_()
    gw[:S].copy_(dx.view(B, S, -1).sum(0))


def head_forward_backward(x: torch.Tensor, targets: torch.Tensor, p: Dict[str, torch.Tensor],
                          gr: Dict[str, torch.Tensor], cfg: GPTConfig, grad_scale: float, loss_sum: torch.Tensor,
                          ce_fwd_bwd: Callable, chunk_tokens: Optional[int] = None,
                          branch: Optional[torch.Tensor] = None, dx_sum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Final layer norm, tied output projection and cross-entropy, forward and backward in
    one sweep over token chunks so the [T, vocab] logits never exist in full.  Adds the
    summed token losses to ``loss_sum``; writes gr["wte"], gr["lnf_*"]; returns dx.  With
    ``branch`` the input is ``x + branch`` (see ``layer_forward_deferred``); ``dx_sum`` receives the
    column sums of the returned dx (see ``layer_backward``)."""
    T, d = x.shape
    if chunk_tokens is None:
        # one chunk while the bf16 logits stay below 2 GiB: then all three products of the head are
        # single launches of the library GEMM (an accumulating second chunk would need cuBLAS)
        chunk_tokens = T if T * cfg.vocab * 2 <= (2 << 30) else 4096
    hf, mean, rstd, x = _ln_fwd(x, p["lnf_w"], p["lnf_b"], cfg.ln_eps, branch)
    wte = p["wte"]
    dhf = torch.empty_like(hf)
    gw = gr["wte"]
    tflat = targets.reshape(-1)
    first = True
    for s in range(0, T, chunk_tokens):
        e = min(T, s + chunk_tokens)
        logits = mm_nt(hf[s:e], wte)                            # [c, V] bf16
        ce_fwd_bwd(logits, tflat[s:e], loss_sum, grad_scale)    # logits -> dlogits, in place
        mm_nn(logits, wte, out=dhf[s:e])
        if first:
            mm_tn(logits, hf[s:e], out=gw)
            first = False
        else:
            gw.addmm_(logits.t(), hf[s:e])                      # later chunks accumulate: cuBLAS
        del logits
    return _ln_bwd(dhf, x, mean, rstd, p["lnf_w"], p["lnf_b"], gr["lnf_w"], gr["lnf_b"], dx_sum=dx_sum)
