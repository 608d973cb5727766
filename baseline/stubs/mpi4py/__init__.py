"""Import stand-in for ``mpi4py`` on machines without an MPI implementation.

Every module of the reference library imports ``mpi4py`` at import time
(``pccl/all_gather.py:7``, ``pccl/process_groups.py:3``, ``pccl/request.py:2``,
``pccl/build_kernels.py:20``), also on code paths that never send an MPI message: its NCCL
branch (``--library xccl``) only needs the names ``MPI.Comm`` and ``MPI.Request`` for
``isinstance`` checks.  This package provides those names so that the unmodified reference
can be imported and its NCCL branch timed.  Anything that would really communicate through
MPI raises.
"""
import os

from . import MPI  # noqa: F401


def get_include() -> str:
    """Where ``mpi4py.h`` would be; nothing here can be compiled against."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "include")
