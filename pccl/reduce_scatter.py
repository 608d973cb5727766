"""Reduce-scatter (SUM): dispatcher, Python ring / recursive halving, and the 2-D form.

Public names and signatures follow ``pccl/reduce_scatter.py`` of the reference
(``recursive_halving_reduce_scatter_mpi`` :20-98, ``ring_reduce_scatter_mpi`` :102-161,
``_reduce_scatter`` :164-203, ``reduce_scatter_2D`` :205-235).  What differs underneath:

* with ``use_pccl_cpp_backend=True`` on a ``pccl.Group`` the call is one sm_100a kernel;
  the sums are formed in fp32 registers while the data moves, so the reference's clone of
  the input, its receive buffer and its ``vectorAdd`` launches per step are gone;
* bf16 / fp16 / fp32 inputs (the reference's native path takes fp32 only,
  ``pccl/src/pccl.cpp:42-45``), optional fp32 output and a fused ``scale`` (the gradient
  averaging that DeepSpeed otherwise does in a separate pass);
* the 2-D form needs no permute pass (:226): the kernels read each block where it is.
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch
import torch.distributed as dist

from . import schedule as sch
from . import tuner
from ._dispatch import algo_from_flags, completed_request, run_native
from .all_gather import _default_group, _native_ok
from .backends import p2p
from .comm import Group
from .request import Request

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _check_op(op) -> None:
    if op is not torch.add and op is not None:
        raise NotImplementedError("only SUM (op=torch.add) is implemented, as in the reference's dispatcher")


def recursive_halving_reduce_scatter_mpi(output_tensor: torch.Tensor, input_tensor: torch.Tensor,
                                         group: Optional[Group] = None, async_op: bool = False,
                                         op: Callable = torch.add):
    assert not async_op, "non-blocking primitives not supported"
    _check_op(op)
    group = _default_group(group)
    assert input_tensor.numel() % group.size == 0, "Input tensor size must be divisible by the number of processes"
    p2p.reduce_scatter(output_tensor, input_tensor, group.transport(), sch.RECURSIVE)


def ring_reduce_scatter_mpi(output_tensor: torch.Tensor, input_tensor: torch.Tensor,
                            group: Optional[Group] = None, async_op: bool = False, op: Callable = torch.add):
    assert not async_op, "non-blocking primitives not supported"
    _check_op(op)
    group = _default_group(group)
    assert input_tensor.numel() % group.size == 0, "Input tensor size must be divisible by the number of processes"
    p2p.reduce_scatter(output_tensor, input_tensor, group.transport(), sch.RING)


def _reduce_scatter(output_tensor: torch.Tensor, input_tensor: torch.Tensor,
                    group: Optional[Union[dist.ProcessGroup, Group]] = None, async_op: bool = False,
                    directly_call_mpi: bool = False, use_rh: bool = False, use_pccl_cpp_backend: bool = False,
                    algorithm: Optional[str] = None, scale: float = 1.0, wire_dtype: Optional[torch.dtype] = None,
                    lanes: Optional[int] = None) -> Optional[Request]:
    if group is None or isinstance(group, dist.ProcessGroup):
        work = dist.reduce_scatter_tensor(output_tensor, input_tensor, op=dist.ReduceOp.SUM, group=group,
                                          async_op=async_op)
        if scale != 1.0:
            if work is not None:
                work.wait()
            output_tensor.mul_(scale)
            return completed_request() if async_op else None
        return Request(work) if work is not None else None
    if not isinstance(group, Group):
        raise TypeError(
            f"Unsupported group type: {type(group)}. Expected torch.distributed.ProcessGroup or pccl.Group.")
    algo = algo_from_flags(algorithm, use_rh)
    if directly_call_mpi:
        algo = sch.DIRECT   # "let the vendor library decide" has no meaning here; direct is the plain schedule
    if use_pccl_cpp_backend and _native_ok(group, output_tensor, input_tensor):
        comm = group.comm
        nbytes = output_tensor.numel() * input_tensor.element_size()
        algo, nl = tuner.choose("reduce_scatter", group.size, nbytes, requested=algo,
                                symmetric_in=comm.is_symmetric(input_tensor), has_multimem=comm.nvls,
                                lanes=lanes, max_lanes=comm.native.max_lanes,
                                eager_capacity=comm.native.eager_capacity if group.gid == 0 else 0)
        if algo == sch.EAGER and wire_dtype == torch.float32 and input_tensor.dtype != torch.float32:
            algo = sch.DIRECT            # fp32 wire doubles the landing bytes: keep the capacity rule simple
        native = comm.native

        def launch():
            native.reduce_scatter(group.gid, [output_tensor], [input_tensor], sch.ALGO_IDS[algo], nl, scale, wire_dtype)

        return run_native(group, async_op, launch,
                          lambda: f"pccl.reduce_scatter {algo} {nbytes}B/rank P={group.size} lanes={nl}",
                          tensors=(output_tensor, input_tensor))
    if algo == sch.AUTO:
        algo = sch.RECURSIVE if sch.is_pow2(group.size) else sch.RING
    p2p.reduce_scatter(output_tensor, input_tensor, group.transport(), algo, scale, wire_dtype)
    return completed_request() if async_op else None


def reduce_scatter(output_tensor: torch.Tensor, input_tensor: torch.Tensor, group=None, async_op: bool = False,
                   algorithm: str = sch.AUTO, scale: float = 1.0, wire_dtype: Optional[torch.dtype] = None,
                   lanes: Optional[int] = None) -> Optional[Request]:
    """Short form: native kernels, algorithm chosen from the tuning table."""
    if isinstance(group, dist.ProcessGroup):
        return _reduce_scatter(output_tensor, input_tensor, group, async_op, scale=scale)
    return _reduce_scatter(output_tensor, input_tensor, _default_group(group), async_op,
                           use_pccl_cpp_backend=True, algorithm=algorithm, scale=scale, wire_dtype=wire_dtype,
                           lanes=lanes)


def reduce_scatter_2D(output_tensor: torch.Tensor, input_tensor: torch.Tensor, group=None, async_op: bool = False,
                      use_rh: bool = False, use_pccl_cpp_backend: bool = False, algorithm: Optional[str] = None,
                      hierarchical: Optional[bool] = None, scale: float = 1.0,
                      lanes: Optional[int] = None) -> Optional[Request]:
    """Rank g of the grid receives the sum of block g of the global-rank-ordered inputs."""
    assert input_tensor.dim() == 1 and output_tensor.dim() == 1, "reduce_scatter_2D only admits 1D tensors"
    assert group is not None, "reduce_scatter_2D needs a ProcessGroups object"
    intra, inter = group.get_world_size()
    assert input_tensor.numel() % (intra * inter) == 0, "input size must be divisible by intra * inter"
    inner, outer = group.get_inner_group(), group.get_outer_group()
    both_native = (isinstance(inner, Group) and isinstance(outer, Group) and use_pccl_cpp_backend
                   and _native_ok(inner, output_tensor, input_tensor))
    if both_native and not hierarchical:
        return _reduce_scatter(output_tensor, input_tensor, group.get_flat_group(), async_op, False, use_rh, True,
                               algorithm, scale, None, lanes)
    n = input_tensor.numel() // (intra * inter)
    if both_native and _hier_fits(inner.comm, input_tensor, n, intra, inter):
        return _reduce_scatter_2d_native(output_tensor, input_tensor, inner, outer, intra, inter, n, async_op,
                                         algo_from_flags(algorithm, use_rh), scale, lanes)
    # Mixed or non-native levels: two blocking calls.  The reference refuses async_op here
    # (pccl/reduce_scatter.py:212); this path runs in order and hands back a request that is already complete.
    # [outer][inner][n] -> [inner][outer][n] so that the inner level scatters contiguous blocks
    permuted = input_tensor.view(inter, intra, -1).transpose(0, 1).reshape(-1)
    intermediate = torch.empty(input_tensor.numel() // intra, device=input_tensor.device, dtype=input_tensor.dtype)
    _reduce_scatter(intermediate, permuted, inner, False, False, use_rh, use_pccl_cpp_backend, algorithm, lanes=lanes)
    _reduce_scatter(output_tensor, intermediate, outer, False, False, use_rh, use_pccl_cpp_backend, algorithm,
                    scale=scale, lanes=lanes)
    return completed_request() if async_op else None


def _hier_fits(comm, inp: torch.Tensor, n: int, intra: int, inter: int) -> bool:
    need = max((intra - 1) * inter * n, (inter - 1) * n) * inp.element_size()
    return need <= comm.native.staging_bytes


def _reduce_scatter_2d_native(out, inp, inner: Group, outer: Group, intra: int, inter: int, n: int, async_op: bool,
                              algo: str, scale: float, lanes: Optional[int]) -> Optional[Request]:
    comm = inner.comm
    native = comm.native
    es = inp.element_size()
    tin, tout = _DT[inp.dtype], _DT[out.dtype]
    a1, l1 = tuner.choose("reduce_scatter", intra, n * inter * es, requested=algo, lanes=lanes, max_lanes=native.max_lanes)
    a2, l2 = tuner.choose("reduce_scatter", inter, n * es, requested=algo, lanes=lanes, max_lanes=native.max_lanes)
    a1 = sch.DIRECT if a1 in (sch.PULL, sch.MULTIMEM, sch.EAGER) else a1
    a2 = sch.DIRECT if a2 in (sch.PULL, sch.MULTIMEM, sch.EAGER) else a2
    mid = torch.empty(inter * n, dtype=inp.dtype, device=inp.device)

    def launch():
        rs2d_inner_call(native, inner.gid, sch.ALGO_IDS[a1], l1, tin, [inp.data_ptr()], [mid.data_ptr()], n, es,
                        intra, inter)
        rs2d_outer_call(native, outer.gid, sch.ALGO_IDS[a2], l2, tin, tout, [mid.data_ptr()], [out.data_ptr()], n, es,
                        out.element_size(), scale)
        if async_op:
            mid.record_stream(torch.cuda.current_stream())

    return run_native(inner, async_op, launch)


def rs2d_inner_call(native, gid: int, algo_id: int, lanes: int, tin: int, in_ptrs, mid_ptrs, n: int, es: int,
                    intra: int, inter: int) -> None:
    """Inner level of the 2-D reduce-scatter: the block for member i' is the ``inter``
    sub-blocks (o', i'), o' = 0..inter-1, of the global-rank-ordered input."""
    native.reduce_scatter_raw(gid, algo_id, lanes, tin, tin, tin, list(in_ptrs), list(mid_ptrs), 0, native.staging_off,
                              n * es, intra * n * es, n, n * es, inter, 1.0)


def rs2d_outer_call(native, gid: int, algo_id: int, lanes: int, tin: int, tout: int, mid_ptrs, out_ptrs, n: int,
                    es: int, out_es: int, scale: float) -> None:
    """Outer level: plain reduce-scatter of the intermediate over the column."""
    native.reduce_scatter_raw(gid, algo_id, lanes, tin, tin, tout, list(mid_ptrs), list(out_ptrs), 0,
                              native.staging_off, n * es, 0, n, n * out_es, 1, scale)
