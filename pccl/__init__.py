"""pccl: a Blackwell-native collective communication library with PCCL's Python API.

The first block re-exports exactly what ``pccl/__init__.py:1-3`` of the reference does;
the rest are this library's additions (short names, communicator, symmetric memory).
"""
from .process_groups import ProcessGroups
from .all_gather import all_gather_2D, _all_gather, recursive_doubling_allgather_mpi
from .reduce_scatter import reduce_scatter_2D, _reduce_scatter, recursive_halving_reduce_scatter_mpi

from .all_gather import all_gather
from .reduce_scatter import reduce_scatter, ring_reduce_scatter_mpi
from .all_reduce import _all_reduce, all_reduce, barrier, broadcast
from .comm import Communicator, Group, get_communicator, init, shutdown
from .errors import PcclError, PcclPoisonedError, PcclTimeoutError
from .request import Request
from . import schedule

__version__ = "0.1.0"


def empty_symmetric(shape, dtype=None):
    """Tensor in the symmetric heap of the default communicator (collective call)."""
    import torch

    return get_communicator().empty(shape, dtype or torch.float32)


def build():
    """Compile (if needed) and load the native extension."""
    from .build_kernels import build as _build

    return _build()


def __getattr__(name):
    if name == "_C":
        from .build_kernels import load

        return load()
    raise AttributeError(f"module 'pccl' has no attribute {name!r}")
