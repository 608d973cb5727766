"""Exception types of the library.

The reference ends the process on any CUDA error (``CUDA_CHECK`` prints and calls
``exit(1)``, ``pccl/include/common.h:8-15``) and hangs forever when a peer is missing.
Here every device-side wait has a time limit, and an expired one becomes an exception.
"""


class PcclError(RuntimeError):
    """Base class of all errors raised by the library."""


class PcclTimeoutError(PcclError):
    """A bounded wait (device flag, p2p message or rendezvous) ran out."""


class PcclPoisonedError(PcclError):
    """The communicator saw a failure earlier and must be recovered before reuse."""
