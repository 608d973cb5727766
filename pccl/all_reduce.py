"""All-reduce (SUM, in place).

Signature of ``_all_reduce`` follows ``pccl/all_reduce.py:21-55`` of the reference.  There
the library path (``use_yacl``) is reduce-scatter into a temporary followed by all-gather
back (``pccl/src/yacl.cpp:146-177``), in an extension that is never built.  Here
``algorithm="ring"`` / ``"recursive"`` (or the reference's flags: ``use_yacl`` with
``use_rh_and_rd`` for recursive halving + doubling, without it for ring) run that same
composition as ONE kernel launch, in place; ``"direct"`` / ``"auto"`` is the two-shot kernel
over the switch (or, with NVLS, ``multimem.ld_reduce`` + ``multimem.st``).
The reference's silent no-op when neither flag is set (:39-49) is not reproduced.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.distributed as dist

from . import schedule as sch
from . import tuner
from ._dispatch import completed_request, run_native
from .all_gather import _default_group, _native_ok
from .backends import p2p
from .comm import Group
from .request import Request


def _all_reduce(input_tensor: torch.Tensor, group: Optional[Union[dist.ProcessGroup, Group]] = None,
                async_op: bool = False, use_rh_and_rd: bool = False, use_yacl: bool = False,
                directly_call_mpi: bool = False, algorithm: Optional[str] = None, scale: float = 1.0,
                lanes: Optional[int] = None) -> Optional[Request]:
    if group is None or isinstance(group, dist.ProcessGroup):
        work = dist.all_reduce(input_tensor, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        if scale != 1.0:
            if work is not None:
                work.wait()
            input_tensor.mul_(scale)
            return completed_request() if async_op else None
        return Request(work) if work is not None else None
    if not isinstance(group, Group):
        raise TypeError(
            f"Unsupported group type: {type(group)}. Expected torch.distributed.ProcessGroup or pccl.Group.")
    native_wanted = use_yacl or directly_call_mpi or algorithm is not None
    if native_wanted and _native_ok(group, input_tensor) and input_tensor.is_contiguous():
        comm = group.comm
        nbytes = input_tensor.numel() * input_tensor.element_size()
        requested = algorithm
        if requested is None and use_yacl:
            # the reference's flags: recursive halving + doubling, else ring (pccl/all_reduce.py:39-42)
            requested = sch.RECURSIVE if (use_rh_and_rd and sch.is_pow2(group.size)) else sch.RING
        algo, nl = tuner.choose("all_reduce", group.size, nbytes // max(1, group.size),
                                requested=requested or sch.AUTO, symmetric_in=comm.is_symmetric(input_tensor),
                                has_multimem=comm.nvls, lanes=lanes, max_lanes=comm.native.max_lanes)
        if algo in (sch.RING, sch.RECURSIVE) and input_tensor.numel() % group.size != 0:
            algo = sch.DIRECT        # the two-phase schedules cut the tensor into equal blocks
        algo_id = sch.ALGO_IDS[algo if algo in (sch.MULTIMEM, sch.RING, sch.RECURSIVE) else sch.DIRECT]
        native = comm.native

        def launch():
            native.all_reduce(group.gid, [input_tensor], algo_id, nl, scale)

        return run_native(group, async_op, launch,
                          lambda: f"pccl.all_reduce {algo} {nbytes}B P={group.size} lanes={nl}", tensors=(input_tensor,))
    algo = algorithm if algorithm in (sch.RING, sch.RECURSIVE, sch.DIRECT) else None
    if algo is None:
        algo = sch.RECURSIVE if (use_rh_and_rd and sch.is_pow2(group.size)) else sch.RING
    p2p.all_reduce(input_tensor, group.transport(), algo, scale)
    return completed_request() if async_op else None


def all_reduce(tensor: torch.Tensor, group=None, async_op: bool = False, algorithm: str = sch.AUTO,
               scale: float = 1.0, lanes: Optional[int] = None) -> Optional[Request]:
    if isinstance(group, dist.ProcessGroup):
        return _all_reduce(tensor, group, async_op, scale=scale)
    return _all_reduce(tensor, _default_group(group), async_op, algorithm=algorithm, scale=scale, lanes=lanes)


def broadcast(tensor: torch.Tensor, src: int, group=None, async_op: bool = False,
              lanes: Optional[int] = None) -> Optional[Request]:
    """``src`` is an index into the group.  Root pushes to every peer in one kernel (or one
    ``multimem.st`` stream); ``pccl/patch_deepspeed.py:78-84`` uses MPI Bcast for this."""
    if isinstance(group, dist.ProcessGroup):
        work = dist.broadcast(tensor, dist.get_global_rank(group, src), group=group, async_op=async_op)
        return Request(work) if work is not None else None
    group = _default_group(group)
    if _native_ok(group, tensor) and tensor.is_contiguous():
        comm = group.comm
        nbytes = tensor.numel() * tensor.element_size()
        nl = lanes or tuner.default_lanes(nbytes, min(comm.native.max_lanes, tuner.DEFAULT_MAX_LANES))
        native = comm.native

        def launch():
            native.broadcast(group.gid, [tensor], src, nl, comm.nvls)

        return run_native(group, async_op, launch, lambda: f"pccl.broadcast root={src} {nbytes}B P={group.size} lanes={nl}",
                          tensors=(tensor,))
    p2p.broadcast(tensor, src, group.transport())
    return completed_request() if async_op else None


def barrier(group=None, async_op: bool = False, host_sync: bool = True) -> Optional[Request]:
    """Device barrier kernel; with ``host_sync`` the host also waits for it, which is the
    meaning of ``torch.cuda.synchronize(); MPI Barrier`` in ``pccl/patch_deepspeed.py:86-93``."""
    if isinstance(group, dist.ProcessGroup):
        work = dist.barrier(group=group, async_op=async_op)
        return Request(work) if work is not None else None
    group = _default_group(group)
    if group.native:
        comm = group.comm
        native = comm.native
        req = run_native(group, async_op, lambda: native.barrier(group.gid), lambda: f"pccl.barrier P={group.size}")
        if host_sync and not async_op:
            comm.check(sync=True)
        return req
    p2p.barrier(group.transport())
    return completed_request() if async_op else None
