"""Device-side timing helpers: CUDA events on the launching stream, max over ranks.

The reference times 20 back-to-back calls with one event pair and reports rank 0's mean
(``benchmark_raw_collectives/utils.py:16-33``, ``.../all_gather.py:106-111``); these helpers
keep that shape (warm-up, then one event pair around the timed calls) but reduce with MAX
over the ranks, because a collective is only as fast as its slowest member.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def max_over_ranks(value: float, group=None) -> float:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


_flush_buf: Optional[torch.Tensor] = None


def flush_l2(nbytes: int = 256 << 20) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    global _flush_buf
    if _flush_buf is None or _flush_buf.numel() < nbytes:
        _flush_buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_something(fn: Callable, *args, warmup_iters: int = 5, timed_iters: int = 20, group=None,
                   flush: bool = False, **kwargs) -> float:
    """Mean milliseconds per call, device-timed, max over ranks.  With ``flush`` every call is
    timed by its own event pair with an L2 flush in between; otherwise one pair brackets
    all calls (inputs are expected to exceed L2)."""
    for i in range(warmup_iters):
        with torch.profiler.record_function(f"warmup_{i}"):
            fn(*args, **kwargs)
    torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)
        torch.cuda.synchronize()
    if flush:
        total = 0.0
        for i in range(timed_iters):
            flush_l2()
            st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record()
            with torch.profiler.record_function(f"iteration_{i}"):
                fn(*args, **kwargs)
            en.record()
            en.synchronize()
            total += st.elapsed_time(en)
        ms = total / timed_iters
    else:
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        for i in range(timed_iters):
            with torch.profiler.record_function(f"iteration_{i}"):
                fn(*args, **kwargs)
        en.record()
        torch.cuda.synchronize()
        ms = st.elapsed_time(en) / timed_iters
    return max_over_ranks(ms, group)
