"""All-gather: dispatcher, Python recursive doubling, and the 2-D hierarchical form.

Public names and signatures follow ``pccl/all_gather.py`` of the reference
(``_all_gather`` :98-134, ``recursive_doubling_allgather_mpi`` :14-93, ``all_gather_2D``
:136-159).  What differs underneath:

* a library group is a ``pccl.Group`` (the reference takes an ``MPI.Comm``); with
  ``use_pccl_cpp_backend=True`` the call is ONE sm_100a kernel that performs every step of
  the chosen schedule over NVLink, instead of a host loop of ``MPI_Sendrecv``;
* "ring" is a real ring all-gather (the reference calls the vendor ``MPI Allgather``
  there, :123-128) and ``algorithm=`` adds ``direct``, ``pull``, ``multimem`` and ``auto``;
* ``async_op=True`` returns a real ``Request``;
* the 2-D form needs no un-permute pass (:158-159): the kernels write every block to its
  final, global-rank-ordered position.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.distributed as dist

from . import schedule as sch
from . import tuner
from ._dispatch import algo_from_flags, completed_request, run_native
from .backends import p2p
from .comm import Group
from .request import Request


def recursive_doubling_allgather_mpi(output_tensor: torch.Tensor, input_tensor: torch.Tensor,
                                     group: Optional[Group] = None, async_op: bool = False):
    """Recursive-doubling all-gather executed from Python over point-to-point messages.
    The name is kept from the reference; the transport is ``torch.distributed`` p2p."""
    assert not async_op, "non-blocking primitives not supported"
    group = _default_group(group)
    assert output_tensor.numel() == group.size * input_tensor.numel(), "Output tensor has incorrect size"
    p2p.all_gather(output_tensor, input_tensor, group.transport(), sch.RECURSIVE)


def _default_group(group):
    if group is not None:
        return group
    from .comm import get_communicator

    return get_communicator().world_group


def _native_ok(group: Group, *tensors: torch.Tensor) -> bool:
    return group.native and all(t.is_cuda for t in tensors)


def _all_gather(output_tensor: torch.Tensor, input_tensor: torch.Tensor,
                group: Optional[Union[dist.ProcessGroup, Group]] = None, async_op: bool = False,
                use_rd: bool = False, use_pccl_cpp_backend: bool = False, algorithm: Optional[str] = None,
                lanes: Optional[int] = None) -> Optional[Request]:
    if group is None or isinstance(group, dist.ProcessGroup):
        work = dist.all_gather_into_tensor(output_tensor, input_tensor, group, async_op)
        return Request(work) if work is not None else None
    if not isinstance(group, Group):
        raise TypeError(
            f"Unsupported group type: {type(group)}. Expected torch.distributed.ProcessGroup or pccl.Group.")
    algo = algo_from_flags(algorithm, use_rd)
    if algo == sch.COPY_ENGINE:
        comm = group.comm
        if not (use_pccl_cpp_backend and _native_ok(group, output_tensor, input_tensor) and not comm.emulated
                and comm.is_symmetric(input_tensor) and output_tensor.is_contiguous() and input_tensor.is_contiguous()):
            raise ValueError("algorithm='copy_engine' needs the native backend, one rank per process and an input "
                             "allocated with pccl.empty_symmetric")
        native = comm.native
        nbytes = input_tensor.numel() * input_tensor.element_size()

        def launch_ce():
            native.all_gather_copy_engine(group.gid, output_tensor, input_tensor)

        return run_native(group, async_op, launch_ce,
                          lambda: f"pccl.all_gather copy_engine {nbytes}B/rank P={group.size}", copy_stream=True,
                          tensors=(output_tensor, input_tensor))
    if use_pccl_cpp_backend and _native_ok(group, output_tensor, input_tensor):
        comm = group.comm
        nbytes = input_tensor.numel() * input_tensor.element_size()
        algo, nl = tuner.choose("all_gather", group.size, nbytes, requested=algo,
                                symmetric_in=comm.is_symmetric(input_tensor),
                                symmetric_out=comm.is_symmetric(output_tensor),
                                has_multimem=comm.nvls, lanes=lanes, max_lanes=comm.native.max_lanes,
                                eager_capacity=comm.native.eager_capacity if group.gid == 0 else 0)
        if algo == sch.MULTIMEM and not comm.is_symmetric(output_tensor):
            algo = sch.DIRECT
        native = comm.native

        def launch():
            native.all_gather(group.gid, [output_tensor], [input_tensor], sch.ALGO_IDS[algo], nl)

        return run_native(group, async_op, launch,
                          lambda: f"pccl.all_gather {algo} {nbytes}B/rank P={group.size} lanes={nl}",
                          tensors=(output_tensor, input_tensor))
    if algo == sch.AUTO:
        algo = sch.RECURSIVE if sch.is_pow2(group.size) else sch.RING
    p2p.all_gather(output_tensor, input_tensor, group.transport(), algo)
    return completed_request() if async_op else None


def all_gather(output_tensor: torch.Tensor, input_tensor: torch.Tensor, group=None, async_op: bool = False,
               algorithm: str = sch.AUTO, lanes: Optional[int] = None) -> Optional[Request]:
    """Short form: native kernels, algorithm chosen from the tuning table."""
    if isinstance(group, dist.ProcessGroup):
        return _all_gather(output_tensor, input_tensor, group, async_op)
    return _all_gather(output_tensor, input_tensor, _default_group(group), async_op,
                       use_pccl_cpp_backend=True, algorithm=algorithm, lanes=lanes)


def all_gather_2D(output_tensor: torch.Tensor, input_tensor: torch.Tensor, group=None, async_op: bool = False,
                  use_rd: bool = False, use_pccl_cpp_backend: bool = False, algorithm: Optional[str] = None,
                  hierarchical: Optional[bool] = None, lanes: Optional[int] = None) -> Optional[Request]:
    """Gather over all ``intra * inter`` ranks of a ``ProcessGroups`` grid; the result is in
    global-rank order.  ``hierarchical=False`` runs one flat kernel over the whole grid
    (on one NVSwitch domain every pair of GPUs is equally close); ``True`` keeps the
    reference's two levels (outer groups first, then inner groups); ``None`` picks flat when
    both levels are native."""
    assert input_tensor.dim() == 1 and output_tensor.dim() == 1, "all_gather_2D only admits 1D tensors"
    assert group is not None, "all_gather_2D needs a ProcessGroups object"
    intra, inter = group.get_world_size()
    inner, outer = group.get_inner_group(), group.get_outer_group()
    both_native = (isinstance(inner, Group) and isinstance(outer, Group) and use_pccl_cpp_backend
                   and _native_ok(inner, output_tensor, input_tensor))
    if both_native and not hierarchical:
        return _all_gather(output_tensor, input_tensor, group.get_flat_group(), async_op, use_rd, True, algorithm, lanes)
    if both_native and _hier_native_fits(inner.comm, output_tensor, input_tensor, intra * inter):
        return _all_gather_2d_native(output_tensor, input_tensor, inner, outer, intra, inter, async_op,
                                     algo_from_flags(algorithm, use_rd), lanes)
    # Mixed or non-native levels: two blocking calls.  The reference refuses async_op here
    # (pccl/all_gather.py:143); this path runs in order and hands back a request that is already complete.
    intermediate = torch.empty(input_tensor.size(0) * inter, device=input_tensor.device, dtype=input_tensor.dtype)
    _all_gather(intermediate, input_tensor, outer, False, use_rd, use_pccl_cpp_backend, algorithm, lanes)
    _all_gather(output_tensor, intermediate, inner, False, use_rd, use_pccl_cpp_backend, algorithm, lanes)
    # inner-major -> global-rank order
    output_tensor.copy_(output_tensor.view(intra, inter, -1).transpose(0, 1).reshape(-1))
    return completed_request() if async_op else None


def _hier_native_fits(comm, out: torch.Tensor, inp: torch.Tensor, total_ranks: int) -> bool:
    if comm.is_symmetric(out):
        return True
    return inp.numel() * inp.element_size() * total_ranks <= comm.native.staging_bytes


def _all_gather_2d_native(out, inp, inner: Group, outer: Group, intra: int, inter: int, async_op: bool,
                          algo: str, lanes: Optional[int]) -> Optional[Request]:
    comm = inner.comm
    native = comm.native
    n = inp.numel() * inp.element_size()
    o, i = outer.rank, inner.rank
    out_off = native.offset_of(out.data_ptr(), out.numel() * out.element_size(), comm.rank)
    recv_off = out_off if out_off >= 0 else native.staging_off
    out_ptr = 0 if out_off >= 0 else out.data_ptr()
    a1, l1 = tuner.choose("all_gather", inter, n, requested=algo, lanes=lanes, max_lanes=native.max_lanes)
    a2, l2 = tuner.choose("all_gather", intra, n * inter, requested=algo, lanes=lanes, max_lanes=native.max_lanes)
    a1 = sch.DIRECT if a1 in (sch.PULL, sch.MULTIMEM, sch.EAGER) else a1
    a2 = sch.DIRECT if a2 in (sch.PULL, sch.MULTIMEM, sch.EAGER) else a2

    def launch():
        ag2d_outer_call(native, outer.gid, sch.ALGO_IDS[a1], l1, [inp.data_ptr()], recv_off, i, n, intra)
        ag2d_inner_call(native, inner.gid, sch.ALGO_IDS[a2], l2, [out_ptr], recv_off, n, intra, inter)

    return run_native(inner, async_op, launch)


def ag2d_outer_call(native, gid: int, algo_id: int, lanes: int, in_ptrs, recv_off: int, inner_index: int, n: int,
                    intra: int) -> None:
    """Outer level of the 2-D all-gather: member o' of column ``inner_index`` lands at block
    ``o'*intra + inner_index`` of the landing zone."""
    native.all_gather_raw(gid, algo_id, lanes, list(in_ptrs), [0] * len(in_ptrs), recv_off + inner_index * n,
                          0, 0, intra * n, 0, n, n, 1, 0)


def ag2d_inner_call(native, gid: int, algo_id: int, lanes: int, out_ptrs, recv_off: int, n: int, intra: int,
                    inter: int) -> None:
    """Inner level, in place: member i' contributes the ``inter`` blocks ``o'*intra + i'``;
    a non-zero ``out_ptrs`` entry receives the whole result in global-rank order."""
    native.all_gather_raw(gid, algo_id, lanes, [0] * len(out_ptrs), list(out_ptrs), recv_off,
                          n, intra * n, n, intra * n, n, n, inter, 0)
