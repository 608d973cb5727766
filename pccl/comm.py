"""Communicator and groups: who the ranks are and how their memory is reached.

A ``Communicator`` owns one symmetric heap per rank, maps every peer's heap and signal pad
into this process, and wraps the native ``_C.Comm`` that launches the collective kernels.
A ``Group`` is an ordered subset of the communicator's ranks; it is what the collectives
take as their ``group`` argument.  It stands where the reference has an ``MPI.Comm`` made
by ``MPI.COMM_WORLD.Split`` (``pccl/process_groups.py:118-139``).

``torch.distributed`` is used only to bootstrap (exchange handles, agree on a transport)
and as the transport of the Python fallback; no collective kernel goes through it.

Bootstrap transports, tried in this order unless ``PCCL_BOOTSTRAP`` names one:

``vmm``       cuMemCreate + POSIX file descriptors passed over unix sockets; the only one
              that can also bind an NVLS multicast object (``PCCL_ENABLE_NVLS=1``).
``ipc``       cudaMalloc + cudaIpc handles passed through ``all_gather_object``.
``symm_mem``  ``torch.distributed._symmetric_memory`` does the mapping.
"""
from __future__ import annotations

import array
import atexit
import os
import socket
import struct
import uuid
import weakref
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import schedule as sch
from .backends.p2p import P2PTransport
from .errors import PcclError, PcclPoisonedError, PcclTimeoutError

_KIND_NAMES = {0: "entry", 1: "exit"}
_COLL_NAMES = {1: "all_gather", 2: "reduce_scatter", 3: "all_reduce", 4: "broadcast", 5: "barrier", 6: "ag_gemm", 7: "wait_probe"}

DEFAULT_HEAP_BYTES = 1 << 30
DEFAULT_SIG_BYTES = 4 << 20
DEFAULT_STAGING_BYTES = 256 << 20
_GUARD_BYTES = 256      # canary bytes on either side of a guarded symmetric tensor
_GUARD_VALUE = 0xA5


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    mult = 1
    v = v.strip()
    for suffix, m in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
        if v.upper().endswith(suffix):
            mult, v = m, v[:-1]
            break
    return int(float(v) * mult)


def _native():
    from . import build_kernels

    return build_kernels.load()


class Group:
    """Ordered list of world ranks with this process's position in it.

    ``native`` is true when collective kernels can run on it (CUDA communicator present);
    otherwise the collectives fall back to the Python algorithms over ``pg`` p2p messages.
    """

    def __init__(self, ranks: Sequence[int], my_world_rank: int, comm: Optional["Communicator"], gid: int,
                 pg=None, p2p_timeout_s: Optional[float] = None):
        self.ranks = list(ranks)
        self.size = len(self.ranks)
        self.rank = self.ranks.index(my_world_rank) if my_world_rank in self.ranks else -1
        self.comm = comm
        self.gid = gid
        self.pg = pg
        self.p2p_timeout_s = p2p_timeout_s

    @property
    def native(self) -> bool:
        return self.comm is not None and self.comm.native is not None

    @property
    def is_member(self) -> bool:
        return self.rank >= 0

    def transport(self) -> P2PTransport:
        return P2PTransport(self.ranks, self.rank, self.pg, self.p2p_timeout_s)

    def Get_rank(self) -> int:   # mpi4py-style accessors, used by code written for the reference
        return self.rank

    def Get_size(self) -> int:
        return self.size

    def __repr__(self) -> str:
        kind = "native" if self.native else "p2p"
        return f"<pccl.Group {kind} ranks={self.ranks} rank={self.rank}>"


class Communicator:
    def __init__(self):
        self.native = None           # _C.Comm
        self.rank = 0
        self.world = 1
        self.device: Optional[int] = None
        self.emulated = False
        self.transport_name = "none"
        self.pg = None
        self._segments: List[Any] = []
        self._keepalive: List[Any] = []
        self._groups: List[Group] = []
        self.world_group: Optional[Group] = None
        self._side_stream = None
        self._guards = os.environ.get("PCCL_DEBUG", "0") == "1"     # canary bytes around symmetric tensors
        self._guarded: List[Any] = []
        self._closed = False
        self.nvls = False

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, pg=None, heap_bytes: Optional[int] = None, staging_bytes: Optional[int] = None,
               sig_bytes: Optional[int] = None, device: Optional[int] = None, transport: Optional[str] = None,
               enable_nvls: Optional[bool] = None, timeout_ms: Optional[float] = None) -> "Communicator":
        """Collective over all ranks of ``pg`` (default: the world).  On a machine without
        CUDA the result has no native part and every collective uses the Python fallback."""
        if not dist.is_initialized():
            raise PcclError("pytorch distributed should be initialized by the user before creating a communicator")
        self = cls()
        self.pg = pg
        self.rank = dist.get_rank(pg)
        self.world = dist.get_world_size(pg)
        p2p_timeout = float(os.environ.get("PCCL_P2P_TIMEOUT_S", "0")) or None
        if not torch.cuda.is_available():
            self.world_group = Group(list(range(self.world)), self.rank, self, 0, pg, p2p_timeout)
            self._groups.append(self.world_group)
            return self
        if self.world > sch.MAX_RANKS:
            raise PcclError(f"a communicator spans one NVSwitch domain: at most {sch.MAX_RANKS} ranks, got {self.world}")
        self.device = torch.cuda.current_device() if device is None else device
        heap_bytes = heap_bytes or _env_int("PCCL_HEAP_BYTES", DEFAULT_HEAP_BYTES)
        staging_bytes = staging_bytes if staging_bytes is not None else _env_int("PCCL_STAGING_BYTES", DEFAULT_STAGING_BYTES)
        sig_bytes = sig_bytes or DEFAULT_SIG_BYTES
        heap_bytes = max(heap_bytes, staging_bytes + (1 << 20))
        if enable_nvls is None:
            enable_nvls = os.environ.get("PCCL_ENABLE_NVLS", "0") == "1" and os.environ.get("PCCL_DISABLE_NVLS", "0") != "1"
        order = [transport or os.environ.get("PCCL_BOOTSTRAP", "auto")]
        if order == ["auto"]:
            order = ["vmm", "ipc", "symm_mem"]
        C = _native()
        errors: Dict[str, str] = {}
        tables = None
        for name in order:
            try:
                tables = getattr(self, f"_bootstrap_{name}")(C, heap_bytes, sig_bytes, enable_nvls)
                self._self_check(C, tables[1], sig_bytes)
                ok, msg = True, ""
            except Exception as exc:  # noqa: BLE001 - every failure means "try the next transport"
                ok, msg = False, f"{type(exc).__name__}: {exc}"
            verdicts: List[Any] = [None] * self.world
            dist.all_gather_object(verdicts, (ok, msg), group=pg)
            if all(v[0] for v in verdicts):
                self.transport_name = name
                break
            errors[name] = "; ".join(f"rank {i}: {v[1]}" for i, v in enumerate(verdicts) if not v[0])
            self._release_segments()
            tables = None
        if tables is None:
            raise PcclError(f"no peer-memory transport could be set up: {errors}")
        heaps, sigs, mc, heap_bytes = tables
        self.nvls = mc != 0
        self.native = C.Comm(self.world, self.rank, 1, self.device, heaps, sigs, mc, heap_bytes, sig_bytes, staging_bytes)
        if timeout_ms is None:
            timeout_ms = float(os.environ.get("PCCL_TIMEOUT_MS", "20000"))
        self.native.set_timeout_ms(timeout_ms)
        jitter_us = float(os.environ.get("PCCL_DEBUG_JITTER_US", "0"))
        trace_events = int(os.environ.get("PCCL_TRACE_EVENTS", "0"))
        if jitter_us > 0 or trace_events > 0:
            self.native.set_debug(int(jitter_us * 1000), trace_events)
        self.world_group = self._register_group(list(range(self.world)), p2p_timeout)
        dist.barrier(group=pg)   # every peer has mapped everything before the first kernel
        atexit.register(_close_weak, weakref.ref(self))
        return self

    @classmethod
    def emulated_world(cls, world: int, device: int = 0, heap_bytes: int = 64 << 20, staging_bytes: int = 16 << 20,
                       timeout_ms: float = 2000.0) -> "Communicator":
        """All ``world`` ranks on ONE GPU: every collective becomes a single cooperative
        launch whose blockIdx.y is the rank.  For tests on a single device."""
        self = cls()
        C = _native()
        self.world, self.rank, self.device, self.emulated = world, 0, device, True
        sig_bytes = DEFAULT_SIG_BYTES
        heaps, sigs = [], []
        for _ in range(world):
            h = torch.zeros(heap_bytes, dtype=torch.uint8, device=f"cuda:{device}")
            s = torch.zeros(sig_bytes, dtype=torch.uint8, device=f"cuda:{device}")
            self._keepalive += [h, s]
            heaps.append(h.data_ptr())
            sigs.append(s.data_ptr())
        torch.cuda.synchronize(device)
        self.native = C.Comm(world, 0, world, device, heaps, sigs, 0, heap_bytes, sig_bytes, staging_bytes)
        self.native.set_timeout_ms(timeout_ms)
        self.transport_name = "emulated"
        self.world_group = self._register_group(list(range(world)), None)
        return self

    @classmethod
    def with_fake_peers(cls, world: int, rank: int = 0, device: int = 0, heap_bytes: int = 8 << 20,
                        staging_bytes: int = 1 << 20, timeout_ms: float = 50.0) -> "Communicator":
        """One real rank whose "peers" are local buffers that nobody drives.  Any collective
        on it must run into its bounded wait: this is how timeouts are tested without a
        second GPU and without hanging the one that is there."""
        self = cls.emulated_world(world, device, heap_bytes, staging_bytes, timeout_ms)
        C = _native()
        heaps = [self.native.heap_base(r) for r in range(world)]
        sig_bytes = DEFAULT_SIG_BYTES
        sigs = [self._keepalive[2 * r + 1].data_ptr() for r in range(world)]
        self.native = C.Comm(world, rank, 1, device, heaps, sigs, 0, heap_bytes, sig_bytes, staging_bytes)
        self.native.set_timeout_ms(timeout_ms)
        self.rank, self.emulated, self.transport_name = rank, False, "fake_peers"
        self._groups = []
        self.world_group = self._register_group(list(range(world)), None)
        return self

    # ------------------------------------------------------------------ bootstrap transports
    def _all_gather_obj(self, obj):
        out: List[Any] = [None] * self.world
        dist.all_gather_object(out, obj, group=self.pg)
        return out

    def _agree(self, fn):
        """Run one bootstrap phase locally, then exchange its result with every rank.
        Each phase ends in exactly one collective, and a failure on ANY rank raises on ALL
        ranks at the same phase, so the ranks never fall out of step while falling back."""
        try:
            res, ok, msg = fn(), True, ""
        except Exception as exc:  # noqa: BLE001
            res, ok, msg = None, False, f"{type(exc).__name__}: {exc}"
        allv = self._all_gather_obj((ok, msg, res))
        bad = [f"rank {i}: {v[1]}" for i, v in enumerate(allv) if not v[0]]
        if bad:
            raise PcclError("; ".join(bad))
        return [v[2] for v in allv]

    def _bootstrap_ipc(self, C, heap_bytes, sig_bytes, enable_nvls):
        def make():
            heap = C.IpcSegment(self.device, heap_bytes)
            sig = C.IpcSegment(self.device, sig_bytes)
            self._segments += [heap, sig]
            return heap.handle(), sig.handle()

        handles = self._agree(make)
        heaps: List[int] = [0] * self.world
        sigs: List[int] = [0] * self.world

        def open_peers():
            heaps[self.rank], sigs[self.rank] = self._segments[0].ptr, self._segments[1].ptr
            for r, (hh, sh) in enumerate(handles):
                if r == self.rank:
                    continue
                ph = C.IpcSegment(self.device, hh, heap_bytes)
                ps = C.IpcSegment(self.device, sh, sig_bytes)
                self._segments += [ph, ps]
                heaps[r], sigs[r] = ph.ptr, ps.ptr

        self._agree(open_peers)
        return heaps, sigs, 0, heap_bytes

    def _bootstrap_vmm(self, C, heap_bytes, sig_bytes, enable_nvls):
        want_mc = bool(enable_nvls) and self.world > 1

        def make():
            mc_ok = want_mc and C.VmmSegment.multicast_supported(self.device)
            heap = C.VmmSegment(self.device, heap_bytes, self.world if mc_ok else 0)
            sig = C.VmmSegment(self.device, sig_bytes, 0)
            self._segments += [heap, sig]
            return heap.bytes, sig.bytes, mc_ok, uuid.uuid4().hex

        made = self._agree(make)
        heap, sig = self._segments[0], self._segments[1]
        if any(m[:2] != made[0][:2] for m in made):
            made = self._agree(lambda: (_ for _ in ()).throw(PcclError(f"segment sizes differ: {made}")))
        use_mc = all(m[2] for m in made)
        job = made[0][3]
        chan_box: List[Any] = []
        heaps: List[int] = [0] * self.world
        sigs: List[int] = [0] * self.world
        try:
            self._agree(lambda: chan_box.append(_FdChannel(job, self.rank, self.world)))
            chan = chan_box[0]

            def exchange():
                for p in range(self.world):
                    if p != self.rank:
                        chan.send(p, [heap.export_fd(), sig.export_fd()], tag=0)
                heaps[self.rank], sigs[self.rank] = heap.ptr, sig.ptr
                for _ in range(self.world - 1):
                    src, tag, fds = chan.recv()
                    if tag != 0 or len(fds) != 2:
                        raise PcclError("unexpected message while exchanging memory handles")
                    ph = C.VmmSegment.from_fd(self.device, fds[0], heap.bytes)
                    ps = C.VmmSegment.from_fd(self.device, fds[1], sig.bytes)
                    self._segments += [ph, ps]
                    heaps[src], sigs[src] = ph.ptr, ps.ptr

            self._agree(exchange)
            mc = 0
            if use_mc:
                def mc_handles():
                    if self.rank == 0:
                        fd = heap.multicast_create(self.world)
                        try:
                            for p in range(1, self.world):
                                chan.send(p, [os.dup(fd)], tag=1)
                        finally:
                            os.close(fd)
                    else:
                        src, tag, fds = chan.recv()
                        if tag != 1 or len(fds) != 1:
                            raise PcclError("unexpected message while exchanging the multicast handle")
                        heap.multicast_import(fds[0])
                    heap.multicast_add_device()

                self._agree(mc_handles)          # binding needs every device added first
                mc = self._agree(heap.multicast_bind_and_map)[self.rank]
        finally:
            for c in chan_box:
                c.close()
        return heaps, sigs, mc, heap.bytes

    def _bootstrap_symm_mem(self, C, heap_bytes, sig_bytes, enable_nvls):
        import torch.distributed._symmetric_memory as symm_mem

        group = self.pg if self.pg is not None else dist.group.WORLD
        buf = symm_mem.empty(heap_bytes + sig_bytes, dtype=torch.uint8, device=f"cuda:{self.device}")
        hdl = symm_mem.rendezvous(buf, group.group_name)
        buf.zero_()
        torch.cuda.synchronize(self.device)
        self._agree(lambda: None)        # nobody writes into a peer before that peer has cleared its memory
        self._keepalive += [buf, hdl]
        ptrs = list(hdl.buffer_ptrs)
        sigs = [int(p) for p in ptrs]
        heaps = [int(p) + sig_bytes for p in ptrs]
        mc = 0
        if enable_nvls and getattr(hdl, "multicast_ptr", 0):
            mc = int(hdl.multicast_ptr) + sig_bytes
        return heaps, sigs, mc, heap_bytes

    def _self_check(self, C, sigs: List[int], sig_bytes: int) -> None:
        """Prove that every mapping reaches the peer's memory: each rank writes a word into the
        tail of every peer's signal pad, then reads its own pad back.  A transport that maps
        but does not deliver fails here, on all ranks together, and the next one is tried."""
        if self.world == 1:
            return
        words = sig_bytes // 4
        magic = 0x50C0FFEE

        def write():
            for p in range(self.world):
                if p != self.rank:
                    C.poke_u32(sigs[p] + 4 * (words - self.world + self.rank), magic + self.rank)

        self._agree(write)

        def read():
            for p in range(self.world):
                if p != self.rank:
                    got = C.peek_u32(sigs[self.rank] + 4 * (words - self.world + p))
                    if got != magic + p:
                        raise PcclError(f"word written by rank {p} did not arrive (read 0x{got:x})")
                    C.poke_u32(sigs[self.rank] + 4 * (words - self.world + p), 0)

        self._agree(read)

    def _release_segments(self) -> None:
        for s in reversed(self._segments):
            try:
                s.close()
            except Exception:  # noqa: BLE001
                pass
        self._segments = []
        self._keepalive = []

    # ------------------------------------------------------------------ groups
    def _register_group(self, ranks: List[int], p2p_timeout) -> Group:
        gid = self.native.new_group(ranks) if self.native is not None else len(self._groups)
        my = self.rank if not self.emulated else ranks[0]
        g = Group(ranks, my, self, gid, self.pg, p2p_timeout)
        self._groups.append(g)
        return g

    def new_group(self, ranks: Optional[Sequence[int]] = None) -> Group:
        """Collective over the whole communicator (like ``dist.new_group``): every rank calls
        it with the same ``ranks``, members and non-members alike."""
        ranks = list(range(self.world)) if ranks is None else list(ranks)
        timeout = self.world_group.p2p_timeout_s if self.world_group else None
        return self._register_group(ranks, timeout)

    # ------------------------------------------------------------------ memory
    def empty(self, shape, dtype=torch.float32):
        """Tensor in the symmetric heap.  Collective: every rank must allocate (and free) the
        same sizes in the same order so that offsets agree.  Emulated communicators return
        one tensor per rank."""
        if self.native is None:
            return torch.empty(shape, dtype=dtype)
        numel = 1
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        for s in shape:
            numel *= s
        nbytes = max(1, numel * torch.empty((), dtype=dtype).element_size())
        guard = _GUARD_BYTES if self._guards else 0
        off = self.native.alloc(nbytes + 2 * guard, 256)
        if off < 0:
            raise PcclError(
                f"symmetric heap exhausted: wanted {nbytes} bytes, {self.native.heap_used} of "
                f"{self.native.heap_bytes} in use (set PCCL_HEAP_BYTES)")
        owners = list(range(self.world)) if self.emulated else [self.rank]
        # the storage of these tensors returns the block to the allocator when it dies
        if not guard:
            tensors = [t.view(shape) for t in self.native.owned_tensors(off, numel, dtype, owners)]
            return tensors if self.emulated else tensors[0]
        # Guarded allocation: 256 canary bytes in front of and behind the tensor.  A kernel that
        # writes outside a buffer by up to 256 bytes changes them, and check_guards() says which
        # buffer it was.  The user's tensor is a view into the middle of the owning byte tensor.
        raw = self.native.owned_tensors(off, nbytes + 2 * guard, torch.uint8, owners)
        tensors = []
        for r, b in zip(owners, raw):
            b[:guard].fill_(_GUARD_VALUE)
            b[guard + nbytes:].fill_(_GUARD_VALUE)
            t = b[guard:guard + numel * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)
            self._guarded.append((weakref.ref(t), r, off, nbytes))
            tensors.append(t)
        return tensors if self.emulated else tensors[0]

    def check_guards(self) -> None:
        """With guard words on (``set_debug(guards=True)`` or ``PCCL_DEBUG=1``): synchronise and
        verify the canary bytes around every live symmetric tensor of this process; raise
        ``PcclError`` naming the first buffer whose surroundings were overwritten."""
        if self.native is None or not self._guarded:
            return
        torch.cuda.synchronize(self.device)
        alive = []
        for ref, r, off, nbytes in self._guarded:
            if ref() is None:
                continue
            alive.append((ref, r, off, nbytes))
            front = self.native.tensor(off, _GUARD_BYTES, torch.uint8, r)
            back = self.native.tensor(off + _GUARD_BYTES + nbytes, _GUARD_BYTES, torch.uint8, r)
            for name, g in (("in front of", front), ("behind", back)):
                if not bool((g == _GUARD_VALUE).all()):
                    bad = int((g != _GUARD_VALUE).nonzero()[0])
                    raise PcclError(f"guard bytes {name} the symmetric tensor at heap offset {off + _GUARD_BYTES} "
                                    f"({nbytes} bytes, rank {r}) were overwritten (first at byte {bad})")
        self._guarded = alive

    def is_symmetric(self, t: torch.Tensor) -> bool:
        if self.native is None or not t.is_cuda:
            return False
        return self.native.offset_of(t.data_ptr(), t.numel() * t.element_size(), self.rank) >= 0

    # ------------------------------------------------------------------ failures
    def check(self, sync: bool = True) -> None:
        """Raise if a kernel of this communicator reported a failure.  ``sync=True`` first
        waits for the device, so every call issued so far has had its say."""
        if self.native is None:
            return
        if sync:
            torch.cuda.synchronize(self.device)
        if not self.native.poisoned():
            return
        n = self.world if self.emulated else 1
        for li in range(n):
            st = self.native.status(li)
            if st["code"] != 0:
                kind = st["slot_kind"]
                kname = _KIND_NAMES.get(kind, f"step{kind - 2}")
                msg = (f"{_COLL_NAMES.get(st['collective'], st['collective'])} call #{st['epoch']}: rank "
                       f"{st['rank']} lane {st['lane']} gave up waiting for the '{kname}' flag of rank {st['peer']} "
                       f"(last value seen {st['seen']}) after {self.native.timeout_ms():.0f} ms")
                if st["code"] == 1:
                    raise PcclTimeoutError(msg)
                raise PcclPoisonedError(msg)

    # ------------------------------------------------------------------ debugging aids
    def set_debug(self, jitter_us: float = 0.0, trace_events: int = 0, guards: Optional[bool] = None) -> None:
        """Stress mode and device-side trace, both off by default.

        ``jitter_us`` > 0: every lane of every kernel of this communicator sleeps a pseudo-random
        time below that before each wait and each signal, so ranks and lanes meet in orders a quiet
        machine never produces; results must not change (the GPU tests run the collectives this
        way against their references).  ``trace_events`` > 0: the kernels record every completed
        wait and published flag (time, call number, rank, lane, flag kind) in device memory;
        ``trace()`` reads them.  Also set from ``PCCL_DEBUG_JITTER_US`` / ``PCCL_TRACE_EVENTS``
        when the communicator is created.  The reference has neither: its only hook is
        ``record_function`` around benchmark iterations (``benchmark_raw_collectives/utils.py:20,27``)."""
        if guards is not None:
            # canary bytes around every symmetric tensor allocated from now on (``PCCL_DEBUG=1`` sets
            # this from the start); ``check_guards()`` verifies them on the host
            self._guards = bool(guards)
        if self.native is None:
            return
        torch.cuda.synchronize(self.device)
        self.native.set_debug(int(jitter_us * 1000), int(trace_events))

    def trace(self):
        """Device-side trace since the last call: ``(events, dropped)`` with one dict per event,
        sorted by time.  Synchronises the device."""
        if self.native is None:
            return [], 0
        rows, dropped = self.native.read_trace()
        events = [{"t_ns": t, "call": epoch, "rank": rank, "lane": lane,
                   "flag": _KIND_NAMES.get(kind, f"step{kind - 2}"), "op": "signal" if sig else "wait",
                   "collective": _COLL_NAMES.get(coll, coll)}
                  for (t, epoch, rank, lane, kind, sig, coll) in rows]
        events.sort(key=lambda e: e["t_ns"])
        return events, int(dropped)

    def recover(self) -> None:
        """Forget a failure.  Every surviving rank must call it at the same point; the host
        barrier makes sure no rank restarts while another still clears its flags."""
        if self.native is None:
            return
        self.native.reset_after_failure()
        if self.transport_name in ("vmm", "ipc", "symm_mem"):
            dist.barrier(group=self.pg)

    def side_stream(self):
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device, priority=-1)
        return self._side_stream

    def copy_stream(self):
        """Second side stream: asynchronous copy-engine transfers go here, so they are not queued
        behind the collective kernels of ``side_stream``."""
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(device=self.device, priority=-1)
        return self._copy_stream

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        if self.device is not None and torch.cuda.is_available():
            try:
                torch.cuda.synchronize(self.device)
            except Exception:  # noqa: BLE001
                pass
        self.native = None
        self._release_segments()

    def __repr__(self) -> str:
        return (f"<pccl.Communicator rank={self.rank}/{self.world} device={self.device} "
                f"transport={self.transport_name} nvls={self.nvls}>")


def _close_weak(ref) -> None:
    comm = ref()
    if comm is not None:
        comm.close()


class _FdChannel:
    """Datagram unix sockets in the abstract namespace, one per rank, carrying file
    descriptors (SCM_RIGHTS) between the processes of one node."""

    def __init__(self, job: str, rank: int, world: int, timeout_s: float = 30.0):
        self.job, self.rank, self.world = job, rank, world
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
        self.sock.settimeout(timeout_s)
        self.sock.bind(self._addr(rank))

    def _addr(self, rank: int) -> str:
        return f"\0pccl-{self.job}-{rank}"

    def send(self, dst: int, fds: List[int], tag: int) -> None:
        try:
            # socket.send_fds drops its address argument, so spell the ancillary message out
            anc = [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", fds))]
            self.sock.sendmsg([struct.pack("ii", self.rank, tag)], anc, 0, self._addr(dst))
        finally:
            for fd in fds:
                os.close(fd)

    def recv(self):
        msg, fds, _flags, _addr = socket.recv_fds(self.sock, 8, 8)
        src, tag = struct.unpack("ii", msg)
        return src, tag, list(fds)

    def close(self) -> None:
        self.sock.close()


# ---------------------------------------------------------------------- module-level default
_default: Optional[Communicator] = None


def init(pg=None, **kwargs) -> Communicator:
    """Create (once) the default communicator over ``pg`` (default: the world)."""
    global _default
    if _default is None or _default._closed:
        _default = Communicator.create(pg, **kwargs)
    return _default


def get_communicator() -> Communicator:
    if _default is None:
        raise PcclError("pccl.init() has not been called")
    return _default


def shutdown() -> None:
    global _default
    if _default is not None:
        _default.close()
        _default = None
