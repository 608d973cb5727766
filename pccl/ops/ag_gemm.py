"""Fused parameter all-gather + GEMM.

``AllGatherLinear`` holds a weight sharded by rows over a group (each rank owns ``N/P``
rows in the symmetric heap).  ``forward(x)`` launches ONE kernel that pulls the peers'
shards over NVLink into a local ``[N, K]`` buffer while it multiplies: output tiles whose
weight rows are local start at once, the others as their 256-row panel lands.  Afterwards
the gathered weight is available in ``w_full`` (the backward pass of a ZeRO-3 step reuses
or re-gathers it).

This is the B200 counterpart of what the reference does at its DeepSpeed hook
(``pccl/patch_deepspeed.py:29-40``): there the gather is a blocking collective and the GEMM
that consumes the parameters starts only after it.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from ..comm import Communicator, Group


def _C():
    from .. import build_kernels

    return build_kernels.load()


def auto_gather_ctas(tokens: int, out_features: int, in_features: int, world: int, per_cta_gbs: float = 9.0,
                     gemm_tflops: float = 1450.0, margin: float = 1.3) -> int:
    """How many CTAs should move shards so that the gather just keeps ahead of the multiply.

    The remote part of the weight, ``(P-1)/P * N * K`` bf16 elements, has to arrive within the
    time the GEMM needs for the whole product; a gatherer CTA moves about ``per_cta_gbs`` GB/s
    over NVLink while the other SMs multiply (9 GB/s measured inside this kernel at two ranks,
    against 20-23 GB/s for the same copy path in a collective that has the GPU to itself), the
    multiplying CTAs sustain about ``gemm_tflops`` together.  Every CTA that gathers is one that does not multiply, so the
    count is the smallest even number that covers the required rate with ``margin``."""
    remote_bytes = (world - 1) / world * out_features * in_features * 2
    t_math = 2.0 * tokens * out_features * in_features / (gemm_tflops * 1e12)
    need = remote_bytes / max(t_math, 1e-9) / (per_cta_gbs * 1e9) * margin
    even = int(math.ceil(need / 2.0)) * 2
    return max(4, min(32, even))


class AllGatherLinear:
    def __init__(self, comm: Communicator, group: Optional[Group], out_features: int, in_features: int,
                 gather_ctas: int = 16, device=None, two_cta: bool = True, copy_engine: bool = False,
                 panels_per_copy: int = 0):
        self.comm = comm
        self.group = group or comm.world_group
        P = self.group.size
        if out_features % (P * 256) != 0:
            raise ValueError(f"out_features must be a multiple of 256 * group size ({256 * P})")
        if in_features % 8 != 0:
            raise ValueError("in_features must be a multiple of 8")
        self.N, self.K, self.P = out_features, in_features, P
        self.gather_ctas = gather_ctas       # 0: sized per call from the shapes (auto_gather_ctas)
        self.two_cta = two_cta       # multiply with CTA pairs (cta_group::2, 256x256 tiles)
        # gather with the GPU's copy engines instead of gatherer CTAs: peer-to-local copies on a
        # second stream plus one stream-ordered flag write per 256-row panel; every SM multiplies.
        # No handshake with the peers: their shards must be complete and unchanged during the call.
        self.copy_engine = copy_engine
        self.panels_per_copy = panels_per_copy   # 0: one copy per peer shard
        self.w_shard = comm.empty((out_features // P, in_features), torch.bfloat16)
        dev = device or self.w_shard.device
        self.w_full = torch.empty((out_features, in_features), dtype=torch.bfloat16, device=dev)

    def forward(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, check: bool = False) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.K)
        g = self.gather_ctas if self.gather_ctas > 0 else auto_gather_ctas(x2.shape[0], self.N, self.K, self.P)
        y, err = _C().ag_gemm(self.comm.native, self.group.gid, x2, self.w_shard, self.w_full, bias, None, g, self.two_cta,
                              self.copy_engine, self.panels_per_copy)
        if check:
            code = int(err.item())
            self.comm.check(sync=False)
            if code != 0:
                raise RuntimeError(f"fused all-gather+GEMM gave up in a bounded wait (code {code})")
        return y.view(*lead, self.N)

    __call__ = forward


def make_linear_fwd(comm: Communicator) -> Callable:
    """Forward hook for ``pccl.models.gpt.layer_forward``: QKV and FC1, the two GEMMs that
    consume freshly gathered weights, run on the tcgen05 kernel; everything else stays on
    the default path."""
    from .gemm import linear

    def linear_fwd(x, w, b, which):
        if which in ("qkv", "fc1") and x.dtype == torch.bfloat16 and w.is_contiguous():
            return linear(x, w, b)
        return torch.nn.functional.linear(x, w, b)

    return linear_fwd
