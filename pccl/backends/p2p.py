"""Python collectives over ``torch.distributed`` point-to-point messages.

This is the library's device-agnostic fallback and its test oracle: the schedules of
``pccl.schedule`` are executed step by step with ``batch_isend_irecv``, on CPU tensors
over gloo or on CUDA tensors over NCCL.  It plays the role that the pure-Python MPI
algorithms play in the reference (``pccl/all_gather.py:14-93``,
``pccl/reduce_scatter.py:20-161``, selected there by ``use_pccl_cpp_backend=False``), but
it keeps partial sums in fp32 and it bounds every wait, so a rank that never shows up
turns into a ``PcclTimeoutError`` instead of a hang.
"""
from __future__ import annotations

import datetime
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import schedule as sch
from ..errors import PcclTimeoutError


def _exchange(send: Optional[torch.Tensor], dst_global: int, recv: Optional[torch.Tensor],
              src_global: int, pg, timeout_s: Optional[float]) -> None:
    ops = []
    if send is not None:
        ops.append(dist.P2POp(dist.isend, send, dst_global, group=pg))
    if recv is not None:
        ops.append(dist.P2POp(dist.irecv, recv, src_global, group=pg))
    if not ops:
        return
    # gloo/NCCL report an expired wait as RuntimeError, and a peer whose process has already gone
    # as RuntimeError too ("connection closed by peer"), sometimes while the operation is being
    # posted.  Only those become PcclTimeoutError: a shape or dtype mismatch, an invalid rank or a
    # tensor on the wrong device is a programming error and must not look like a lost peer to code
    # that recovers from lost peers.
    try:
        works = dist.batch_isend_irecv(ops)
        for w in works:
            if timeout_s is None:
                w.wait()
            else:
                w.wait(datetime.timedelta(seconds=timeout_s))
    except RuntimeError as exc:
        if _looks_like_lost_peer(exc):
            raise PcclTimeoutError(
                f"p2p step with dst={dst_global} src={src_global} did not complete: {exc}"
            ) from exc
        raise


_LOST_PEER_MARKS = ("timed out", "timeout", "time out", "connection closed", "connection reset", "connection refused",
                    "broken pipe", "socket closed", "peer closed", "remote process exited", "heartbeat",
                    "application timeout", "watchdog")


def _looks_like_lost_peer(exc: BaseException) -> bool:
    """The messages gloo and NCCL use for an expired wait or a peer whose process is gone."""
    if isinstance(exc, getattr(dist, "DistBackendError", ())) and "invalid" not in str(exc).lower():
        return True
    text = str(exc).lower()
    return any(mark in text for mark in _LOST_PEER_MARKS)


class P2PTransport:
    """Group-index <-> global-rank mapping plus the torch.distributed group to send on."""

    def __init__(self, ranks: Sequence[int], my_index: int, pg=None, timeout_s: Optional[float] = None):
        self.ranks = list(ranks)
        self.rank = my_index
        self.size = len(self.ranks)
        self.pg = pg
        self.timeout_s = timeout_s

    def sendrecv(self, send, dst, recv, src):
        _exchange(send, self.ranks[dst], recv, self.ranks[src], self.pg, self.timeout_s)


def all_gather(out: torch.Tensor, inp: torch.Tensor, tr: P2PTransport, algo: str = sch.RING) -> None:
    P, r = tr.size, tr.rank
    n = inp.numel()
    if out.numel() != P * n:
        raise ValueError(f"output has {out.numel()} elements, expected {P}*{n}")
    if algo in (sch.PULL, sch.MULTIMEM, sch.EAGER):
        algo = sch.DIRECT
    sch.check_algo(algo, P)
    blocks = out.view(-1).view(P, n)
    if blocks[r].data_ptr() != inp.data_ptr():
        blocks[r].copy_(inp.view(-1))
    for t in range(sch.num_steps(algo, P)):
        s = sch.ag_step(algo, P, r, t)
        send = blocks[s.send_first:s.send_first + s.nblocks]
        recv = blocks[s.recv_first:s.recv_first + s.nblocks]
        tr.sendrecv(send, s.dst, recv, s.src)


def reduce_scatter(out: torch.Tensor, inp: torch.Tensor, tr: P2PTransport, algo: str = sch.RING,
                   scale: float = 1.0, wire_dtype: Optional[torch.dtype] = None) -> None:
    """SUM reduce-scatter with fp32 accumulation; ``out = cast(scale * sum)``."""
    P, r = tr.size, tr.rank
    if inp.numel() % P != 0:
        raise ValueError(f"input numel {inp.numel()} is not divisible by the group size {P}")
    n = inp.numel() // P
    if out.numel() != n:
        raise ValueError(f"output has {out.numel()} elements, expected {n}")
    if algo in (sch.PULL, sch.MULTIMEM, sch.EAGER):
        algo = sch.DIRECT
    sch.check_algo(algo, P)
    wire = wire_dtype or inp.dtype
    blocks = inp.view(-1).view(P, n)
    nsteps = sch.num_steps(algo, P)
    staged: List[torch.Tensor] = []      # what arrived at step j
    recv_first: List[int] = []

    def partial(b: int, t: int) -> torch.Tensor:
        acc = blocks[b].to(torch.float32)
        for j in sch.rs_dep_steps(algo, P, t):
            lo = recv_first[j]
            if lo <= b < lo + staged[j].shape[0]:
                acc = acc + staged[j][b - lo].to(torch.float32)
        return acc

    for t in range(nsteps):
        s = sch.rs_step(algo, P, r, t)
        payload = torch.stack([partial(b, t) for b in range(s.send_first, s.send_first + s.nblocks)]).to(wire)
        landing = torch.empty((s.nblocks, n), dtype=wire, device=inp.device)
        tr.sendrecv(payload, s.dst, landing, s.src)
        staged.append(landing)
        recv_first.append(s.recv_first)
    res = partial(r, nsteps)
    if scale != 1.0:
        res = res * scale
    out.view(-1).copy_(res.to(out.dtype))


def all_reduce(t: torch.Tensor, tr: P2PTransport, algo: str = sch.RING, scale: float = 1.0) -> None:
    """In-place all-reduce as reduce-scatter followed by all-gather
    (the composition of ``pccl/src/yacl.cpp:146-177`` in the reference), padding when the
    element count is not a multiple of the group size."""
    P = tr.size
    flat = t.view(-1)
    n = flat.numel()
    per = (n + P - 1) // P
    if per * P != n:
        work = torch.zeros(per * P, dtype=t.dtype, device=t.device)
        work[:n].copy_(flat)
    else:
        work = flat
    piece = torch.empty(per, dtype=t.dtype, device=t.device)
    reduce_scatter(piece, work, tr, algo, scale)
    all_gather(work, piece, tr, algo)
    if work is not flat:
        flat.copy_(work[:n])


def broadcast(t: torch.Tensor, src: int, tr: P2PTransport) -> None:
    """Root pushes to every peer (the switch gives each pair full bandwidth)."""
    if tr.size == 1:
        return
    if tr.rank == src:
        for d in range(tr.size):
            if d != src:
                _exchange(t, tr.ranks[d], None, 0, tr.pg, tr.timeout_s)
    else:
        _exchange(None, 0, t, tr.ranks[src], tr.pg, tr.timeout_s)


def barrier(tr: P2PTransport) -> None:
    """Dissemination barrier: ceil(log2 P) rounds of one-word messages."""
    P, r = tr.size, tr.rank
    # the tokens live where the group's backend can send them from: the device for NCCL, the host for gloo
    on_gpu = dist.is_initialized() and dist.get_backend(tr.pg) == "nccl" and torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
    token = torch.zeros(1, dtype=torch.int32, device=dev)
    got = torch.zeros(1, dtype=torch.int32, device=dev)
    d = 1
    while d < P:
        tr.sendrecv(token, (r + d) % P, got, (r - d) % P)
        d *= 2
