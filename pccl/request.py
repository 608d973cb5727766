"""Handle of a non-blocking collective.

Parity with ``pccl/request.py:6-80`` of the reference: ``Request(handle).wait(epilogue)``
waits, then calls ``epilogue()`` with no arguments, and ``backend`` names the kind of
handle.  The reference wraps ``torch.distributed.Work`` or ``mpi4py.MPI.Request`` and never
actually constructs one (every collective there is synchronous and its DeepSpeed hook
returns a dummy object).  Here a request is real: kernels launched on a side stream are
represented by a CUDA event, and ``wait`` makes the *current stream* wait for it, which is
the stream-ordered meaning ``torch.distributed`` gives to ``Work.wait()`` on CUDA.
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch
import torch.distributed as dist


class Request:
    def __init__(self, request: Any, comm: Any = None):
        if isinstance(request, dist.Work):
            self.backend = "torch"
        elif isinstance(request, torch.cuda.Event):
            self.backend = "pccl"
        elif request is None or getattr(request, "_pccl_completed", False):
            self.backend = "completed"   # synchronous host-side work (CPU fallback) already done
        elif _is_mpi_request(request):
            self.backend = "mpi"
        else:
            raise ValueError(
                f"Unsupported request type: {type(request)}. "
                "Expected torch.distributed.Work, torch.cuda.Event or mpi4py.MPI.Request."
            )
        self.request = request
        self._comm = comm

    def is_completed(self) -> bool:
        if self.backend == "torch":
            return self.request.is_completed()
        if self.backend == "pccl":
            return self.request.query()
        if self.backend == "mpi":
            return self.request.Test()
        return True

    def wait(self, epilogue: Optional[Callable[[], None]] = None) -> Optional[Any]:
        result = None
        if self.backend == "torch":
            self.request.wait()
        elif self.backend == "pccl":
            torch.cuda.current_stream().wait_event(self.request)
            if self._comm is not None:
                self._comm.check(sync=False)
        elif self.backend == "mpi":
            from mpi4py import MPI  # only reachable when mpi4py exists

            result = MPI.Status()
            self.request.Wait(result)
        if epilogue is not None:
            if not callable(epilogue):
                raise TypeError("Epilogue must be a callable.")
            epilogue()
        return result

    def synchronize(self) -> None:
        """Block the host until the work is done (``wait`` only orders the stream)."""
        if self.backend == "pccl":
            self.request.synchronize()
            if self._comm is not None:
                self._comm.check(sync=False)
        else:
            self.wait()

    def __repr__(self) -> str:
        return f"<Request backend={self.backend} request={self.request}>"


def _is_mpi_request(obj: Any) -> bool:
    try:
        from mpi4py import MPI
    except Exception:
        return False
    return isinstance(obj, MPI.Request)
