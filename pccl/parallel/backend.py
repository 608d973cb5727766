"""The five-method communication backend that a ZeRO-3 engine talks to.

DeepSpeed routes every collective through ``deepspeed.comm.torch.TorchBackend``; the
reference hooks exactly that method table (``pccl/patch_deepspeed.py:108-126``).  DeepSpeed
is not a dependency of this library, so this module provides a class with the same
method names and signatures.  The in-repo ZeRO-3 engine calls it, and
``pccl.patch_deepspeed.patch_deepspeed`` patches it (and DeepSpeed's own class too when
DeepSpeed is importable).  Unpatched, every method is plain ``torch.distributed`` (NCCL on
GPUs): that is the baseline arm.
"""
from __future__ import annotations

import torch.distributed as dist


class TorchBackend:
    """Same public surface as DeepSpeed's ``TorchBackend`` for the calls ZeRO-3 makes."""

    def __init__(self, name: str = "torch"):
        self.name = name

    def all_gather_into_tensor(self, output_tensor, input_tensor, group=None, async_op=False):
        return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)

    def reduce_scatter_tensor(self, output_tensor, input_tensor, op=dist.ReduceOp.SUM, group=None, async_op=False):
        return dist.reduce_scatter_tensor(output_tensor, input_tensor, op=op, group=group, async_op=async_op)

    def all_reduce(self, tensor, op=dist.ReduceOp.SUM, group=None, async_op=False):
        return dist.all_reduce(tensor, op=op, group=group, async_op=async_op)

    def broadcast(self, tensor, src, group=None, async_op=False):
        return dist.broadcast(tensor, src, group=group, async_op=async_op)

    def barrier(self, group=dist.GroupMember.WORLD, async_op=False, device_ids=None):
        return dist.barrier(group=group, async_op=async_op, device_ids=device_ids)

    # capability flags the engine consults; patch_deepspeed flips them on the class
    fused_scale = False          # reduce_scatter_tensor accepts scale= and a float32 output
    symmetric_memory = False     # buffers should come from pccl.empty_symmetric
