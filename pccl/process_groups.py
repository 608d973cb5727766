"""2-D Cartesian grid of process groups.

Same constructor, accessors and rank layout as ``pccl/process_groups.py:11-263`` of the
reference: the world is cut into ``num_2d_grids x inter x intra`` with ``np.arange(world)
.reshape(grids, inter, intra)`` semantics, inner groups are runs of consecutive ranks,
outer groups are ranks ``intra`` apart.  Each level independently names its backend.

What differs: the reference's levels are "nccl" (``dist.new_group``) or "mpi"
(``MPI.COMM_WORLD.Split``), by default NCCL inside a node and MPI across nodes.  Here both
levels default to "pccl", this library's own groups: inside one NVSwitch domain the
intra/inter split is purely logical.  "nccl" and "gloo" still give torch.distributed
groups (the baseline path); "mpi" is accepted only where mpi4py can be imported.
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch.distributed as dist

from .comm import Communicator, Group, init as _init_default

_BACKENDS = ("pccl", "nccl", "gloo", "mpi")


class ProcessGroups:
    def __init__(self, intra_group_size: int, inter_group_size: int, inner_group_backend: str = "pccl",
                 outer_group_backend: str = "pccl", comm: Optional[Communicator] = None):
        assert dist.is_initialized() or comm is not None, "pytorch distributed should be initialized by the user"
        self.intra_group_size = intra_group_size
        self.inter_group_size = inter_group_size
        self.inner_group_backend = inner_group_backend
        self.outer_group_backend = outer_group_backend
        self._comm = comm
        self.flat_group = None
        self.inner_group, self.outer_group = self.create_2D_grid(
            intra_group_size, inter_group_size, inner_group_backend, outer_group_backend, _owner=self)

    @staticmethod
    def create_2D_grid(intra_group_size: int, inter_group_size: int, inner_group_backend: str = "pccl",
                       outer_group_backend: str = "pccl", _owner: Optional["ProcessGroups"] = None
                       ) -> List[Union[dist.ProcessGroup, Group]]:
        for b in (inner_group_backend, outer_group_backend):
            if b not in _BACKENDS:
                raise ValueError(f"Unsupported backend {b!r}: expected one of {_BACKENDS}")
            if b == "mpi":
                try:
                    import mpi4py  # noqa: F401
                except ImportError as exc:
                    raise ValueError("backend 'mpi' needs mpi4py, which is not installed here") from exc
                raise ValueError("backend 'mpi' is not wired into this build: use 'pccl' (default), 'nccl' or 'gloo'")
        comm = _owner._comm if _owner is not None else None
        needs_comm = "pccl" in (inner_group_backend, outer_group_backend)
        if needs_comm and comm is None:
            comm = _init_default()
            if _owner is not None:
                _owner._comm = comm
        if comm is not None:
            world, rank = comm.world, comm.rank
        else:
            world, rank = dist.get_world_size(), dist.get_rank()
        if intra_group_size < 1 or inter_group_size < 1 or world % (intra_group_size * inter_group_size) != 0:
            raise ValueError(
                f"world size {world} is not divisible by intra*inter = {intra_group_size}*{inter_group_size}")
        grids = world // (intra_group_size * inter_group_size)

        def world_rank(g: int, o: int, i: int) -> int:
            return (g * inter_group_size + o) * intra_group_size + i

        emulated = comm is not None and comm.emulated
        my_inner = my_outer = my_flat = None
        inner_all, outer_all, flat_all = [], [], []
        # Every rank creates every group, in the same order (group creation is collective).
        for g in range(grids):
            for o in range(inter_group_size):
                ranks = [world_rank(g, o, i) for i in range(intra_group_size)]
                grp = _make_group(ranks, inner_group_backend, comm)
                inner_all.append(grp)
                if rank in ranks:
                    my_inner = grp
        for g in range(grids):
            for i in range(intra_group_size):
                ranks = [world_rank(g, o, i) for o in range(inter_group_size)]
                grp = _make_group(ranks, outer_group_backend, comm)
                outer_all.append(grp)
                if rank in ranks:
                    my_outer = grp
        if needs_comm and inner_group_backend == outer_group_backend == "pccl":
            for g in range(grids):
                ranks = [world_rank(g, o, i) for o in range(inter_group_size) for i in range(intra_group_size)]
                grp = comm.new_group(ranks)
                flat_all.append(grp)
                if rank in ranks:
                    my_flat = grp
        if _owner is not None:
            _owner.flat_group = my_flat
            _owner.num_2d_grids = grids
            _owner.all_inner_groups, _owner.all_outer_groups, _owner.all_flat_groups = inner_all, outer_all, flat_all
            _owner._emulated = emulated
        return [my_inner, my_outer]

    # -------------------------------------------------------------- accessors (reference API)
    def _pair(self, fn):
        return [fn(self.inner_group), fn(self.outer_group)]

    def get_rank(self, idx: Optional[int] = None):
        ranks = self._pair(_group_rank)
        return _select(ranks, idx)

    def get_world_size(self, idx: Optional[int] = None):
        sizes = self._pair(_group_size)
        return _select(sizes, idx)

    def get_inner_group(self):
        return self.inner_group

    def get_outer_group(self):
        return self.outer_group

    def get_flat_group(self):
        """All ranks of this rank's grid in global-rank order (only when both levels are
        "pccl"): the group on which the 2-D collectives run as one flat kernel."""
        if self.flat_group is None:
            raise ValueError("a flat group exists only when both levels use the 'pccl' backend")
        return self.flat_group

    def __repr__(self) -> str:
        return (f"ProcessGroups(inner_group_backend={self.inner_group_backend}, "
                f"outer_group_backend={self.outer_group_backend}, "
                f"rank={self.get_rank()}, world_size={self.get_world_size()})")


def _make_group(ranks: List[int], backend: str, comm: Optional[Communicator]):
    if backend == "pccl":
        return comm.new_group(ranks)
    return dist.new_group(ranks=ranks, backend=backend)


def _group_rank(g) -> int:
    return g.rank if isinstance(g, Group) else dist.get_rank(g)


def _group_size(g) -> int:
    return g.size if isinstance(g, Group) else dist.get_world_size(g)


def _select(pair: List[int], idx: Optional[int]):
    if idx is None:
        return pair
    if idx in (0, 1):
        return pair[idx]
    raise ValueError("idx must be 0 (inner), 1 (outer) or None")
