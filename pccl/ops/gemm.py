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
