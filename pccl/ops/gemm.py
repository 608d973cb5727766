"""Linear layers on the hand-written tcgen05 GEMM (``pccl/csrc/gemm_sm100.cu``).

``linear(x, w, b)`` computes ``x @ w.T + b`` for bf16 operands with fp32 accumulation in
tensor memory.  The reference contains no GEMM; this exists because the ZeRO-3 path fuses
the parameter all-gather with the GEMM that consumes the gathered weight
(``pccl.ops.ag_gemm``), and the fused kernel is this kernel plus gatherer CTAs.
"""
from __future__ import annotations

from typing import Optional

import torch


def _C():
    from .. import build_kernels

    return build_kernels.load()


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           check: bool = False) -> torch.Tensor:
    """x: [..., K] bf16, w: [N, K] bf16, b: [N] bf16 or None.  ``check=True`` synchronises and
    raises if one of the kernel's bounded waits ran out."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y, err = _C().gemm(x2, w, b, out)
    if check and int(err.item()) != 0:
        raise RuntimeError(f"tcgen05 GEMM gave up in a bounded wait (code {int(err.item())})")
    return y.view(*lead, w.shape[0])
