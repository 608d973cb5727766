"""Shared plumbing of the collective entry points: algorithm naming, async launch."""
from __future__ import annotations

import os
from typing import Callable, Optional, Sequence

import torch

from . import schedule as sch
from .comm import Group
from .request import Request


def algo_from_flags(algorithm: Optional[str], recursive_flag: bool) -> str:
    """The reference selects with booleans (``use_rd`` / ``use_rh``: recursive, else ring);
    ``algorithm`` is this library's wider choice and wins when given."""
    if algorithm is not None:
        if algorithm not in (sch.AUTO, sch.COPY_ENGINE) and algorithm not in sch.ALGO_IDS:
            raise ValueError(f"unknown algorithm {algorithm!r}")
        return algorithm
    return sch.RECURSIVE if recursive_flag else sch.RING


# NVTX range around every native collective launch (name, algorithm, bytes, group size, lanes), for
# timeline tools; off unless PCCL_NVTX=1 or this flag is set.  The reference's only ranges are the
# record_function wrappers of its benchmark loop (benchmark_raw_collectives/utils.py:20,27).
NVTX = os.environ.get("PCCL_NVTX", "0") == "1"


def run_native(group: Group, async_op: bool, launch: Callable[[], None],
               label: Optional[Callable[[], str]] = None, copy_stream: bool = False,
               tensors: Sequence[torch.Tensor] = ()) -> Optional[Request]:
    """Enqueue ``launch()`` on the current stream, or, for ``async_op``, on the
    communicator's side stream after everything the current stream has queued so far.
    ``copy_stream``: an asynchronous call goes to the communicator's second side stream, the one
    for copy-engine transfers, so that it is not queued behind collective kernels."""
    comm = group.comm
    if NVTX and label is not None:
        inner, name = launch, label()

        def launch():
            torch.cuda.nvtx.range_push(name)
            try:
                inner()
            finally:
                torch.cuda.nvtx.range_pop()
    if not async_op:
        launch()
        return None
    cur = torch.cuda.current_stream(comm.device)
    side = comm.copy_stream() if copy_stream else comm.side_stream()
    side.wait_stream(cur)
    for t in tensors:
        if t.is_cuda and not comm.is_symmetric(t):      # heap tensors are not the caching allocator's
            t.record_stream(side)
    with torch.cuda.stream(side):
        launch()
        ev = torch.cuda.Event()
        ev.record(side)
    return Request(ev, comm)


class _Done:
    _pccl_completed = True


def completed_request() -> Request:
    return Request(_Done())
