"""Route a ZeRO-3 engine's collectives through this library.

Same entry point and hook set as ``pccl/patch_deepspeed.py:95-126`` of the reference:
``patch_deepspeed(intra_node_pg_size)`` builds the extension, creates the global
``ProcessGroups(intra, world // intra)`` and replaces five methods of the backend class
(``all_gather_into_tensor``, ``reduce_scatter_tensor``, ``all_reduce``, ``broadcast``,
``barrier``), keeping the originals as ``old_*``.  A call is intercepted only when its
group spans the world (and, for reductions, when the op is SUM); anything else goes to
the saved original.

What differs:

* the patched class is DeepSpeed's ``TorchBackend`` when DeepSpeed can be imported, and
  always this library's stand-in ``pccl.parallel.backend.TorchBackend``;
* the reference's hooks block the host and hand back a dummy handle whose ``wait`` does
  nothing (:18-23,37-38), which forfeits DeepSpeed's prefetch overlap; these return real
  stream-ordered ``Request`` objects;
* all-reduce and broadcast run through this library's kernels instead of
  ``MPI.COMM_WORLD.Allreduce`` / ``Bcast`` on a synchronised stream (:61-84);
* ``reduce_scatter_tensor`` accepts ``scale=`` so the gradient averaging is fused.
"""
from __future__ import annotations

from typing import List, Optional

import torch.distributed as dist

from .all_gather import all_gather_2D
from .all_reduce import _all_reduce, barrier as _barrier, broadcast as _broadcast
from .build_kernels import build, build_rank0_first  # noqa: F401  (build: name kept from the reference module)
from .process_groups import ProcessGroups
from .reduce_scatter import reduce_scatter_2D

pg: Optional[ProcessGroups] = None
_patched_classes: List[type] = []


def get_heir_pg() -> ProcessGroups:
    assert pg is not None, "did you call the patch_deepspeed function?"
    return pg


def is_global_pg(group) -> bool:
    return (group is None) or (group == dist.group.WORLD) or (dist.get_world_size(group) == dist.get_world_size())


def _is_sum(op) -> bool:
    if op == dist.ReduceOp.SUM:
        return True
    name = getattr(op, "name", None)       # deepspeed.comm.reduce_op.ReduceOp is its own enum
    return name == "SUM"


def patched_all_gather(self, output_tensor, input_tensor, group=None, async_op=False):
    if is_global_pg(group):
        return all_gather_2D(output_tensor.view(-1), input_tensor.view(-1), group=get_heir_pg(), async_op=async_op,
                             use_rd=True, use_pccl_cpp_backend=True, algorithm=_algo, lanes=_lanes)
    return self.old_all_gather_into_tensor(output_tensor, input_tensor, group, async_op)


def patched_reduce_scatter(self, output_tensor, input_tensor, op=dist.ReduceOp.SUM, group=None, async_op=False,
                           scale: float = 1.0):
    if is_global_pg(group) and _is_sum(op):
        return reduce_scatter_2D(output_tensor.view(-1), input_tensor.view(-1), group=get_heir_pg(), async_op=async_op,
                                 use_rh=True, use_pccl_cpp_backend=True, algorithm=_algo, scale=scale, lanes=_lanes)
    assert scale == 1.0, "scale= is only fused on the library path"
    return self.old_reduce_scatter_tensor(output_tensor, input_tensor, op, group, async_op)


def patched_all_reduce(self, tensor, op=dist.ReduceOp.SUM, group=None, async_op=False):
    if is_global_pg(group) and _is_sum(op) and tensor.is_contiguous():
        return _all_reduce(tensor, get_heir_pg().get_flat_group(), async_op, algorithm="auto")
    return self.old_all_reduce(tensor, op, group, async_op)


def patched_broadcast(self, tensor, src, group=None, async_op=False):
    if is_global_pg(group) and tensor.is_contiguous():
        return _broadcast(tensor, src, get_heir_pg().get_flat_group(), async_op)
    return self.old_broadcast(tensor, src, group, async_op)


def patched_barrier(self, group=dist.GroupMember.WORLD, async_op=False, device_ids=None):
    if is_global_pg(group):
        return _barrier(get_heir_pg().get_flat_group(), async_op, host_sync=True)
    return self.old_barrier(group, async_op, device_ids)


_algo: Optional[str] = None
_lanes: Optional[int] = None

_HOOKS = (
    ("all_gather_into_tensor", patched_all_gather),
    ("reduce_scatter_tensor", patched_reduce_scatter),
    ("all_reduce", patched_all_reduce),
    ("broadcast", patched_broadcast),
    ("barrier", patched_barrier),
)


def _backend_classes() -> List[type]:
    from .parallel.backend import TorchBackend as Ours

    classes = [Ours]
    try:
        from deepspeed.comm.torch import TorchBackend as Theirs   # type: ignore

        classes.append(Theirs)
    except Exception:  # noqa: BLE001 - DeepSpeed is optional
        pass
    return classes


def patch_deepspeed(intra_node_pg_size: int, algorithm: Optional[str] = "auto",
                    lanes: Optional[int] = None) -> ProcessGroups:
    """``algorithm``: "auto" (tuning table; default), or a fixed variant; ``None`` keeps the
    reference's choice (recursive doubling / halving).  ``lanes`` caps the number of SMs a
    parameter gather or gradient reduction may occupy: inside a training step the collectives
    overlap with GEMMs, and a few lanes that leave the other SMs to the math beat many lanes
    that finish the transfer sooner."""
    assert dist.is_initialized()
    assert dist.get_world_size() % intra_node_pg_size == 0
    build_rank0_first(dist.barrier)
    global pg, _algo, _lanes
    _algo = algorithm
    _lanes = lanes
    if pg is None:
        pg = ProcessGroups(intra_node_pg_size, dist.get_world_size() // intra_node_pg_size)
    for cls in _backend_classes():
        if cls in _patched_classes:
            continue
        for name, fn in _HOOKS:
            setattr(cls, "old_" + name, getattr(cls, name))
            setattr(cls, name, fn)
        cls.fused_scale = True
        cls.symmetric_memory = True
        _patched_classes.append(cls)
    return pg


def unpatch_deepspeed() -> None:
    """Restore the saved originals (the reference has no way back)."""
    while _patched_classes:
        cls = _patched_classes.pop()
        for name, _fn in _HOOKS:
            setattr(cls, name, getattr(cls, "old_" + name))
            delattr(cls, "old_" + name)
        cls.fused_scale = False
        cls.symmetric_memory = False
