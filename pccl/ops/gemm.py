"""Linear layers on the hand-written tcgen05 GEMM (``pccl/csrc/gemm_sm100.cu``).

``linear(x, w, b)`` computes ``x @ w.T + b`` for bf16 operands with fp32 accumulation in
tensor memory.  The reference contains no GEMM; this exists because the ZeRO-3 path fuses
the parameter all-gather with the GEMM that consumes the gathered weight
(``pccl.ops.ag_gemm``), and the fused kernel is this kernel plus gatherer CTAs.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _C():
    from .. import build_kernels

    return build_kernels.load()


def _rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.is_contiguous() else x2.contiguous()


def _raise_if(err: torch.Tensor) -> None:
    code = int(err.item())
    if code != 0:
        raise RuntimeError(f"tcgen05 GEMM gave up in a bounded wait (code {code})")


def check_errors(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any GEMM launched on ``device`` since the last reset gave up in
    a bounded wait.  All launches of a device share one error word, so this is one read."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    word = _C().gemm_error_word(idx)
    code = int(word.item())
    if code != 0:
        _C().gemm_reset_error(idx)
        raise RuntimeError(f"a tcgen05 GEMM gave up in a bounded wait (code {code})")


def usable(*ts: torch.Tensor) -> bool:
    """Operands the kernel takes: contiguous 2-D bf16 CUDA tensors on 16-byte boundaries."""
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.is_contiguous() and t.data_ptr() % 16 == 0
               for t in ts)


def matmul_nt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M,K] @ w[N,K]^T (+ bias)``: the forward product of a linear layer."""
    return _C().gemm_ex(a, w, False, False, bias, out)


def matmul_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M,K] @ b[K,N]``: the data gradient ``dy @ W`` of a linear layer with ``W`` stored
    [out_features, in_features]; ``b`` is read as it lies in memory, no transposing copy."""
    return _C().gemm_ex(a, b, False, True, None, out)


def matmul_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[K,M]^T @ b[K,N]``: the weight gradient ``dy^T @ x`` of a linear layer, both operands
    stored [tokens, features] and read as they lie in memory."""
    return _C().gemm_ex(a, b, True, True, None, out)


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           check: bool = False, two_cta: bool = True) -> torch.Tensor:
    """x: [..., K] bf16, w: [N, K] bf16, b: [N] bf16 or None.  ``two_cta`` picks the CTA-pair
    form (``cta_group::2``, one 256x256 tile per pair of SMs; the faster one) over the one-CTA
    form.  ``check=True`` synchronises and raises if one of the kernel's bounded waits ran out."""
    y, err = _C().gemm(_rows(x), w, b, out, two_cta)
    if check:
        _raise_if(err)
    return y.view(*x.shape[:-1], w.shape[0])


def linear_gelu(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, check: bool = False,
                two_cta: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``u = x @ w.T + b`` and ``gelu(u)`` (tanh form) from one kernel: the activation runs in
    the GEMM's epilogue on the accumulator that is being stored anyway.  Returns ``(u, gelu(u))``;
    a backward pass needs both."""
    u, g, err = _C().gemm_gelu(_rows(x), w, b, two_cta)
    if check:
        _raise_if(err)
    lead = x.shape[:-1]
    return u.view(*lead, w.shape[0]), g.view(*lead, w.shape[0])
