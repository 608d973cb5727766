"""A ZeRO-3 (fully sharded data parallel) training engine for the GPT models.

The reference re-routes DeepSpeed's ZeRO-3 collectives (``pccl/patch_deepspeed.py:29-59``)
but contains no engine; DeepSpeed is not a dependency here, so this is the engine that
the hooks serve.  It talks to a backend object with DeepSpeed's five method names
(``pccl.parallel.backend.TorchBackend``): unpatched, that is ``torch.distributed`` over
NCCL (the baseline arm); after ``pccl.patch_deepspeed.patch_deepspeed`` the very same
engine gathers parameters and reduces gradients through this library's kernels.

Memory plan (per rank, P ranks, N parameters):
  bf16 parameter shard N/P, fp32 master + Adam moments 12 N/P, gradient shard 2-4 N/P,
  two rotating gathered-parameter buffers and two rotating gradient buffers of the
  largest unit (bf16), one dedicated gradient buffer for the embedding unit.
With the patched backend all communication buffers live in the symmetric heap, so
all-gathers write straight into the peers' buffers and nothing is staged.

Step schedule: the parameters are cut into units (embedding+final norm, then one unit per
transformer block).  Forward walks the units, prefetching unit k+1 on the communication
stream while unit k computes; the head re-gathers the embedding; backward walks the
blocks in reverse, re-gathering each unit, and hands every unit's gradient buffer to an
asynchronous reduce-scatter as soon as its backward is done.  The optimizer is one fused
AdamW kernel over the whole shard, with global-norm clipping computed on the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..models import gpt
from ..models.gpt import GPTConfig
from .backend import TorchBackend


def _wait(handle) -> None:
    if handle is not None:
        handle.wait()


class _Handles:
    """Several asynchronous collectives that are waited for together."""

    def __init__(self, handles):
        self.handles = [h for h in handles if h is not None]

    def wait(self) -> None:
        for h in self.handles:
            h.wait()


def unit_regions(unit: gpt.UnitSpec, world: int, fused: bool):
    """Cut a unit's flat parameter space into regions that are sharded separately.

    Normally a unit is one region, split evenly over the ranks.  With the fused
    all-gather+GEMM the QKV and FC1 weights are regions of their own, sharded by ROWS, so
    that the fused kernel can gather exactly one weight; everything else is the third
    region.  Returns [(offset, length)] in the gathered layout; lengths are multiples of
    256 * world."""
    gran = world * 256
    pad = lambda n: (n + gran - 1) // gran * gran  # noqa: E731
    names = {p.name: p for p in unit.params}
    if not fused or "qkv_w" not in names:
        return [(0, pad(unit.numel))]
    qkv, fc1 = names["qkv_w"], names["fc1_w"]
    assert qkv.offset == 0 and fc1.offset == qkv.numel, "fused layout expects qkv_w then fc1_w at the front of the unit"
    assert qkv.numel % gran == 0 and fc1.numel % gran == 0
    rest = fc1.offset + fc1.numel
    return [(0, qkv.numel), (fc1.offset, fc1.numel), (rest, pad(unit.numel - rest))]


@dataclass
class OptimConfig:
    lr: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0


def heap_bytes_needed(cfg: GPTConfig, world: int, fused: bool = False) -> int:
    """Symmetric-heap bytes the engine allocates for ``cfg`` on ``world`` ranks (without
    the communicator's staging area)."""
    units = gpt.unit_specs(cfg)
    padded = [sum(r[1] for r in unit_regions(u, world, fused)) for u in units]
    total_shard = sum(n // world for n in padded)
    max_layer = max(padded[1:]) if len(padded) > 1 else padded[0]
    elems = total_shard + 2 * max(padded) + 2 * max_layer + padded[0]
    return 2 * elems + (64 << 20)


class Zero3Engine:
    def __init__(self, cfg: GPTConfig, backend: Optional[TorchBackend] = None, optim: Optional[OptimConfig] = None,
                 device: Optional[torch.device] = None, seed: int = 1234, comm=None, group=None,
                 linear_fwd: Optional[Callable] = None, micro_batch: int = 1, fused_ag_gemm: bool = False,
                 gather_ctas: int = 16, fused_gelu_gemm: bool = False, overlap_wgrad: bool = False,
                 native_gemm: bool = False, copy_engine_gather: bool = False, fused_gelu_bwd_gemm: bool = False,
                 dynamic_tiles: Optional[bool] = None):
        from .. import build_kernels

        self.C = build_kernels.load()
        self.cfg = cfg
        self.backend = backend or TorchBackend()
        self.optim = optim or OptimConfig()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.comm = comm
        self.linear_fwd = linear_fwd or gpt._default_linear
        # True: every dense product of the model on the library's tcgen05 GEMM.  False (default): the
        # plain products on cuBLAS through torch, which was measured 7 % faster per training step, and
        # only the fused products that are switched on (fused_ag_gemm, fused_gelu_gemm) on the library's kernel
        self.native_gemm = bool(native_gemm)
        # The library GEMM hands its tiles out at run time instead of dealing them out in advance.  Default:
        # on when other ranks exist, because then gradient reductions hold some SMs while the backward GEMMs
        # run, and CTA pairs that start late would otherwise work through a full share alone.
        self.dynamic_tiles = (self.world > 1) if dynamic_tiles is None else bool(dynamic_tiles)
        # GELU backward as the epilogue of the data-gradient GEMM of FC2 (needs native_gemm)
        self.fused_gelu_bwd_gemm = bool(fused_gelu_bwd_gemm) and self.native_gemm
        # parameter gathers by the GPU's copy engines instead of gather kernels (no SM is taken from
        # the GEMMs they overlap); needs symmetric parameter shards
        self.copy_engine_gather = bool(copy_engine_gather)
        # FC1 on the library's tcgen05 GEMM with bias and GELU in its epilogue (one kernel, two outputs)
        self.fused_gelu_gemm = bool(fused_gelu_gemm)
        # weight-gradient GEMMs on a second stream, beside the memory-bound kernels of the backward chain
        self.overlap_wgrad = bool(overlap_wgrad)
        self._wgrad_stream = None
        self.micro_batch = micro_batch
        self.step_count = 0
        self.launches = 0          # kernels of this library launched by the last step
        self.units = gpt.unit_specs(cfg)
        P = self.world
        # the fused kernel wants every rank to own whole 256-row panels of the QKV and FC1 weights
        rows_ok = (3 * cfg.d_model) % (P * 256) == 0 and cfg.d_ff % (P * 256) == 0 and cfg.d_model % 8 == 0
        self.fused_ag_gemm = bool(fused_ag_gemm) and rows_ok and P > 1 and comm is not None and \
            comm.native is not None and bool(getattr(self.backend, "symmetric_memory", False))
        self.gather_ctas = gather_ctas
        # regions[ui] = [(offset, length)] in the gathered layout; a unit's shard is the
        # concatenation of its regions' shards
        self.regions = [unit_regions(u, P, self.fused_ag_gemm) for u in self.units]
        self.padded = [rg[-1][0] + rg[-1][1] for rg in self.regions]
        self.shard_len = [sum(l for _o, l in rg) // P for rg in self.regions]
        self.region_shard_off = []       # offset of each region's shard inside the unit's shard
        for rg in self.regions:
            offs, acc = [], 0
            for _o, l in rg:
                offs.append(acc)
                acc += l // P
            self.region_shard_off.append(offs)
        self.shard_off = [0]
        for n in self.shard_len:
            self.shard_off.append(self.shard_off[-1] + n)
        total_shard = self.shard_off[-1]
        max_unit = max(self.padded)
        max_layer = max(self.padded[1:]) if len(self.padded) > 1 else self.padded[0]
        sym = bool(getattr(self.backend, "symmetric_memory", False)) and comm is not None and comm.native is not None
        self.symmetric = sym

        def alloc(n: int) -> torch.Tensor:
            if sym:
                return comm.empty(n, torch.bfloat16)
            return torch.empty(n, dtype=torch.bfloat16, device=self.device)

        self.param_shard = alloc(total_shard)
        # One rank owns everything: the "gathered" parameters are the shard itself and the
        # gradient buffers are the gradient shard, so there is nothing to gather or reduce.
        self.local_only = P == 1
        self.fused_scale = bool(getattr(self.backend, "fused_scale", False)) and not self.local_only
        gdt = torch.float32 if self.fused_scale else torch.bfloat16
        self.grad_shard = torch.zeros(total_shard, dtype=gdt, device=self.device)
        if self.local_only:
            self.gathered, self.gradbuf, self.gradbuf0 = [], [], None
        else:
            self.gathered = [alloc(max_unit), alloc(max_unit)]
            self.gradbuf = [alloc(max_layer), alloc(max_layer)]
            self.gradbuf0 = alloc(self.padded[0])
            for b in self.gradbuf + [self.gradbuf0]:
                b.zero_()
        self.master = torch.empty(total_shard, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros(total_shard, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(total_shard, dtype=torch.float32, device=self.device)
        self.sq_norm = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.loss_sum = torch.zeros(1, dtype=torch.float32, device=self.device)
        # rows whose target was neither the ignore index nor a valid class (the loss kernel skips them)
        self.bad_targets = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._init_params(seed)
        # views of every unit in each rotating buffer
        if self.local_only:
            def unit_of(buf, ui):
                return buf[self.shard_off[ui]: self.shard_off[ui + 1]]

            self.pviews = [[gpt.views(u, unit_of(self.param_shard, ui))] * 2 for ui, u in enumerate(self.units)]
            self.gviews = [None] + [[gpt.views(u, unit_of(self.grad_shard, ui))] * 2
                                    for ui, u in enumerate(self.units) if ui > 0]
            self.gviews0 = gpt.views(self.units[0], unit_of(self.grad_shard, 0))
        else:
            self.pviews = [[gpt.views(u, buf) for buf in self.gathered] for u in self.units]
            self.gviews = [None] + [[gpt.views(u, buf) for buf in self.gradbuf] for u in self.units[1:]]
            self.gviews0 = gpt.views(self.units[0], self.gradbuf0)
        self.main = torch.cuda.current_stream(self.device)
        self._cur = None
        self._dx_sums = None
        self._fused_gid = None
        self._flat_group = None
        self.copy_engine_gather = self.copy_engine_gather and sym and P > 1
        if self.fused_ag_gemm or self.copy_engine_gather:
            from ..patch_deepspeed import get_heir_pg

            self._flat_group = get_heir_pg().get_flat_group()
            self._fused_gid = self._flat_group.gid
        if self.fused_ag_gemm:
            self.linear_fwd = self._fused_linear
        if self.copy_engine_gather:
            # the copy-engine gathers have no handshake with the peers: every rank's shard must be
            # complete before anybody reads it
            dist.barrier(group=group)
        self._rs_pending: List = [None, None]
        self._tokens_dev: Optional[torch.Tensor] = None
        self._targets_dev: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ setup
    def _init_params(self, seed: int) -> None:
        P, r = self.world, self.rank
        for ui, u in enumerate(self.units):
            full = torch.empty(self.padded[ui], dtype=torch.float32, device=self.device)
            gpt.init_unit(u, full, self.cfg, seed + ui)
            for (g_off, g_len), s_off in zip(self.regions[ui], self.region_shard_off[ui]):
                mine = full[g_off:g_off + g_len].view(P, -1)[r]
                lo = self.shard_off[ui] + s_off
                self.master[lo:lo + g_len // P].copy_(mine)
                self.param_shard[lo:lo + g_len // P].copy_(mine)
            del full
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ communication
    def _region_shard(self, buf: torch.Tensor, ui: int, ri: int) -> torch.Tensor:
        lo = self.shard_off[ui] + self.region_shard_off[ui][ri]
        return buf[lo: lo + self.regions[ui][ri][1] // self.world]

    def _gather(self, ui: int, slot: int, skip=()):
        """Start the all-gather of unit ``ui`` into rotating buffer ``slot`` (one collective per
        region; ``skip`` names regions that a fused all-gather+GEMM will fetch itself)."""
        if self.local_only:
            return None
        hs = []
        for ri, (g_off, g_len) in enumerate(self.regions[ui]):
            if ri in skip:
                continue
            out = self.gathered[slot][g_off: g_off + g_len]
            if self.copy_engine_gather:
                from ..all_gather import all_gather as pccl_all_gather
                from .. import schedule as sch

                hs.append(pccl_all_gather(out, self._region_shard(self.param_shard, ui, ri), group=self._flat_group,
                                          async_op=True, algorithm=sch.COPY_ENGINE))
                continue
            hs.append(self.backend.all_gather_into_tensor(out, self._region_shard(self.param_shard, ui, ri),
                                                          group=self.group, async_op=True))
        return hs[0] if len(hs) == 1 else _Handles(hs)

    def _reduce(self, ui: int, buf: torch.Tensor):
        """Start the reduce-scatter of unit ``ui``'s gradient buffer into the gradient shard."""
        if self.local_only:
            return None
        hs = []
        for ri, (g_off, g_len) in enumerate(self.regions[ui]):
            inp = buf[g_off: g_off + g_len]
            out = self._region_shard(self.grad_shard, ui, ri)
            if self.fused_scale:
                hs.append(self.backend.reduce_scatter_tensor(out, inp, group=self.group, async_op=True,
                                                             scale=1.0 / self.world))
            else:
                hs.append(self.backend.reduce_scatter_tensor(out, inp, group=self.group, async_op=True))
        return hs[0] if len(hs) == 1 else _Handles(hs)

    def _fused_linear(self, x, w, b, which):
        """Forward hook for QKV / FC1 of the layer being computed: ONE kernel gathers the
        weight's row shards over NVLink into its place in the gathered buffer and multiplies."""
        if which not in ("qkv", "fc1") or self._cur is None:
            return torch.nn.functional.linear(x, w, b)
        li, slot = self._cur
        ri = 0 if which == "qkv" else 1
        n_rows, k = w.shape
        shard = self._region_shard(self.param_shard, li, ri).view(n_rows // self.world, k)
        gid = self._fused_gid
        y, _err = self.C.ag_gemm(self.comm.native, gid, x, shard, w, b, None, self.gather_ctas, True,
                                 self.copy_engine_gather, 0)
        return y

    # ------------------------------------------------------------------ one training step
    @torch.no_grad()
    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """tokens, targets: [B, S] int64, on the host (pinned) or on the device.  Runs
        forward, backward, gradient reduction and the optimizer; returns the mean loss of
        this rank's micro-batch as a one-element device tensor."""
        cfg, C = self.cfg, self.C
        if tokens.device.type != "cuda":
            if self._tokens_dev is None or self._tokens_dev.shape != tokens.shape:
                self._tokens_dev = torch.empty(tokens.shape, dtype=torch.int64, device=self.device)
                self._targets_dev = torch.empty(targets.shape, dtype=torch.int64, device=self.device)
            self._tokens_dev.copy_(tokens, non_blocking=True)
            self._targets_dev.copy_(targets, non_blocking=True)
            tokens, targets = self._tokens_dev, self._targets_dev
        B, S = tokens.shape
        T = B * S
        L = cfg.n_layer
        launches0 = self._native_launches() + gpt.native_launches
        self.loss_sum.zero_()
        self.sq_norm.zero_()
        # without a fused scale in the reduce-scatter the 1/P of the average rides on the loss gradient
        grad_scale = 1.0 / T if self.fused_scale else 1.0 / (T * self.world)

        # ---- forward
        stage = 0
        pending = self._gather(0, 0)
        nxt = self._gather(1, 1, (0, 1) if self.fused_ag_gemm else ()) if L > 0 else None
        _wait(pending)
        x = gpt.embed_forward(tokens, self.pviews[0][0])
        branch = None          # MLP output of the previous block; the next layer norm adds it to x in its own pass
        gpt.fused_gelu_gemm = self.fused_gelu_gemm
        gpt.native_gemm = self.native_gemm
        C.gemm_set_dynamic_tiles(self.dynamic_tiles)
        gpt.fused_gelu_bwd_gemm = self.fused_gelu_bwd_gemm
        saved = []
        for li in range(1, L + 1):
            slot = li % 2
            _wait(nxt)
            # the buffer that the next prefetch overwrites was last read by the previous stage,
            # which is already queued on this stream; the async launch orders itself after it
            skip = (0, 1) if self.fused_ag_gemm else ()
            nxt = self._gather(li + 1, 1 - slot, skip) if li < L else self._gather(0, 1 - slot)
            self._cur = (li, slot)
            x, branch, ctx = gpt.layer_forward_deferred(x, branch, self.pviews[li][slot], cfg, B, self.linear_fwd)
            self._cur = None
            saved.append(ctx)
        # ---- head: final norm, tied projection, loss; forward and backward together
        head_slot = (L + 1) % 2
        _wait(nxt)
        nxt = self._gather(L, 1 - head_slot) if L > 0 else None
        # every kernel that produces a block's output gradient also sums its columns: that is the
        # FC2 bias gradient of the block, handed down through two small buffers
        if self._dx_sums is None:
            self._dx_sums = [torch.empty(cfg.d_model, dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        dx = gpt.head_forward_backward(x, targets, self.pviews[0][head_slot], self.gviews0, cfg, grad_scale,
                                       self.loss_sum, self._ce, branch=branch, dx_sum=self._dx_sums[L % 2] if L > 0 else None)
        del branch
        # ---- backward through the blocks
        wgrad_stream = None
        if self.overlap_wgrad:
            if self._wgrad_stream is None:
                self._wgrad_stream = torch.cuda.Stream(device=self.device)
            wgrad_stream = self._wgrad_stream
        for li in range(L, 0, -1):
            slot = li % 2
            _wait(nxt)
            nxt = self._gather(li - 1, 1 - slot) if li > 1 else None
            gslot = li % 2
            _wait(self._rs_pending[gslot])          # the buffer's previous reduce-scatter has read it
            dx = gpt.layer_backward(dx, saved.pop(), self.pviews[li][slot], self.gviews[li][gslot], cfg, B,
                                    dy_sum=self._dx_sums[li % 2], dx_sum=self._dx_sums[(li - 1) % 2] if li > 1 else None,
                                    side=wgrad_stream)
            self._rs_pending[gslot] = self._reduce(li, None if self.local_only else self.gradbuf[gslot])
        gpt.embed_backward(dx, tokens, self.gviews0)
        rs0 = self._reduce(0, self.gradbuf0)
        for h in self._rs_pending + [rs0]:
            _wait(h)
        self._rs_pending = [None, None]

        # ---- optimizer: global-norm clipping on the device, then one fused AdamW launch
        self.step_count += 1
        o = self.optim
        if o.max_grad_norm > 0:
            C.sq_norm(self.grad_shard, self.sq_norm)
            if self.world > 1:
                _wait(self.backend.all_reduce(self.sq_norm, group=self.group, async_op=False))
        C.adamw(self.master, self.exp_avg, self.exp_avg_sq, self.grad_shard, self.param_shard, o.lr, o.beta1, o.beta2,
                o.eps, o.weight_decay, self.step_count, 1.0, o.max_grad_norm,
                self.sq_norm if o.max_grad_norm > 0 else None)
        if self.copy_engine_gather:
            # the next step's copy-engine gathers read the peers' shards without a handshake: nobody
            # may start them before every rank's optimizer has written its shard (device barrier
            # kernel on this stream; the host does not wait)
            from ..all_reduce import barrier as pccl_barrier

            pccl_barrier(self._flat_group, host_sync=False)
        ce_chunks = 1 if T * cfg.vocab * 2 <= (2 << 30) else (T + 4095) // 4096
        own = 2 + (1 if o.max_grad_norm > 0 else 0) + ce_chunks  # norm, AdamW, loss kernel per chunk of the head
        self.launches = own + (self._native_launches() + gpt.native_launches - launches0)
        return self.loss_sum / T

    def check_errors(self) -> None:
        """Synchronise and raise if a kernel of the last steps gave up in a bounded wait."""
        torch.cuda.synchronize(self.device)
        from ..ops.gemm import check_errors as check_gemm_errors

        check_gemm_errors(self.device)
        bad = int(self.bad_targets.item())
        if bad:
            self.bad_targets.zero_()
            raise ValueError(f"{bad} target ids were outside [0, {self.cfg.vocab}) and not the ignore index; "
                             "their rows were left out of the loss")
        if self.comm is not None:
            self.comm.check(sync=False)

    def _ce(self, logits, targets, loss_sum, grad_scale) -> None:
        self.C.ce_fwd_bwd(logits, targets, loss_sum, grad_scale, -100, self.bad_targets)

    def _native_launches(self) -> int:
        if self.comm is not None and self.comm.native is not None:
            return int(self.comm.native.kernels_launched)
        return 0

    # ------------------------------------------------------------------ checkpoint (sharded)
    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "step": torch.tensor(self.step_count), "world": torch.tensor(self.world)}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        if int(sd["world"]) != self.world:
            raise ValueError("sharded checkpoint was written with a different world size")
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.param_shard.copy_(self.master)
        self.step_count = int(sd["step"])
