"""Fully sharded data parallelism (``-fsdp``) over peer-mapped memory on one NVSwitch node.

Units and pieces are those of ``sharded.UnitShardedStep``: every encoder / decoder layer is a unit, everything else
(embeddings, final norms, output projection) forms resident units, and rank r keeps piece r of every unit.  What a
rank holds between steps is, per parameter, 1/N of: the bf16 value (in the symmetric heap, where peers read it), the
fp32 master weight, the two Adam moments and the reduced fp32 gradient - 18/N bytes.  Nothing of full size survives
a step except the buffers below:

* **parameter staging**: two rotating buffers, each as large as the largest layer, plus one buffer per resident
  unit.  A layer's weight MATRICES are pulled from their owners by the GEMM that consumes them: the kernel
  (``csrc/gemm2cta_tcgen05.cu``) is told where every piece of the matrix lives, its otherwise idle epilogue warps
  copy the pieces with peer loads into the staging buffer in the order the tiles need them, and its TMA producer
  waits for a segment's completion counter before it loads tiles from that segment - gather and matrix product
  are one launch, the transfer hidden under the tiles already in flight.  Forward uses the weight as a K-major
  operand (``x W^T``), backward as an MN-major one (``dy W``); both gather.  The small parameters of a layer
  (biases, LayerNorm) arrive through one stand-alone copy launch when the layer is entered.  ``fused_gather=False``
  (or ``NMTG_FSDP_FUSED_GATHER=0``) moves everything through the copy kernel one layer ahead on a side stream, the
  unfused baseline.
* **gradient staging**: three rotating fp32 buffers of layer size plus one per resident unit, all in the symmetric
  heap.  When the backward pass leaves a layer, that unit's ``reduce_unit`` launch (communication stream, overlapped
  with the layers below) reduce-scatters the buffer into the owned piece of ``reduced``, tells the peers that it has
  finished reading, and clears the buffer once all peers have; the layer three positions further down then reuses it.
* the fp32 master weights that back ``param.data`` are released after the shards are cut (``param.data`` becomes a
  stride-0 view of a NaN scalar, so an op that bypasses the fused path is noticed immediately) and are
  re-materialised by ``gather_master`` only while a checkpoint is written.

The gather kernels need no flags (shards only change inside ``update_pieces``, which every rank enters after the
step's last gather, and the step ends with a barrier); every cross-GPU wait is bounded and reports through the
status word.

Reference behaviour: FSDP wrapping of the encoder / decoder layers, onmt/train_utils/mp_trainer.py:314-341, and
whisper/train_whisper.py:597-600.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops
from .sharded import Unit, UnitShardedStep, _round_up, plan_units
from .symmetric import SymmetricHeap

GRAD_SLOTS = 3
MIN_FUSED_ELEMS = 1 << 16     # smaller matrices travel with the layer's small parameters


class GatherInfo:
    """Where the pieces of one weight matrix live; attached to the parameter as ``_fsdp`` and handed to the GEMM."""

    __slots__ = ("owner", "unit", "offset", "numel", "valid_key", "used")

    def __init__(self, owner, unit: Unit, offset: int, numel: int):
        self.owner, self.unit, self.offset, self.numel = owner, unit, offset, numel
        self.valid_key = None     # (slot occupancy stamp) for which the staging copy is current
        self.used = False         # some GEMM asked for this matrix during the first step

    def pending(self):
        """Gather arguments if the staging copy of this matrix is stale, else None (marks it current)."""
        return self.owner._claim(self)


class FullyShardedAdam(UnitShardedStep):
    """Sharded parameters + gradients + optimiser state with gather-on-demand staging; plugs into
    ``Optim.attach_distributed``."""

    mode = 1

    def __init__(self, model, store, optim, heap: SymmetricHeap, grad_ptrs=None, gather_ctas: int = 32,
                 fused_gather: Optional[bool] = None, overlap: bool = True):
        assert store.work is None and store.grad is None, "the flat store must be built without full bf16 / gradient buffers"
        world = heap.world
        dev = store.device
        units = plan_units(model, store, world)
        layer_units = [u for u in units if u.slot >= 0]
        # gradient space: [resident units ... | GRAD_SLOTS rotating layer buffers]
        off = 0
        for u in units:
            if u.slot < 0:
                u.grad_base = off
                off += _round_up(u.piece * world, 64)
        self.slot_len = _round_up(max([u.piece * world for u in layer_units], default=64), 64)
        self.gslot_base = [off + i * self.slot_len for i in range(GRAD_SLOTS)]
        for i, u in enumerate(reversed(layer_units)):      # backward order
            u.gslot = i % GRAD_SLOTS
            u.grad_base = self.gslot_base[u.gslot]
        self.grad_len = off + GRAD_SLOTS * self.slot_len if layer_units else max(off, 64)
        self.grad_space, grad_ptrs = heap.alloc(self.grad_len, torch.float32)
        self.shard_len_ = sum(u.piece for u in units)
        self.shard, shard_ptrs = heap.alloc(self.shard_len_, torch.bfloat16)
        self._setup(model, store, optim, heap, grad_ptrs, shard_ptrs, units, overlap=overlap)
        self.shard_ptrs = shard_ptrs
        self.gather_ctas = gather_ctas
        if fused_gather is None:
            fused_gather = os.environ.get("NMTG_FSDP_FUSED_GATHER", "1") != "0"
        self.fused_gather = bool(fused_gather)
        self.master_shard = torch.zeros(self.shard_len, dtype=torch.float32, device=dev)
        self._init_shards()
        # staging: two rotating buffers for layer units, one persistent buffer per resident unit
        self.staging = [torch.zeros(self.slot_len, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.resident = {u.name: torch.zeros(_round_up(u.piece * world, 64), dtype=torch.bfloat16, device=dev)
                         for u in units if u.slot < 0}
        # per staging buffer: completion counters of the in-kernel gathers (cleared by the kernel that used them)
        self.gather_counters = torch.zeros(2, 4096 + 8, dtype=torch.int32, device=dev)
        # First step: every layer is copied whole while the GEMM calls that carry a gather record are noted; matrices
        # that no such call consumed (a layer type that reads its weights some other way) keep travelling with the
        # layer's small parameters afterwards.
        self._learning = self.fused_gather
        self._point_views()
        self._release_master()
        self.side = torch.cuda.Stream(device=dev)
        self.slot_unit = [None, None]          # which unit each staging buffer holds (or is being filled with)
        self.slot_stamp = [0, 0]               # bumped whenever a buffer changes hands
        self.slot_ready = [None, None]         # event: stand-alone gather into the slot finished
        self.gslot_free = [None] * GRAD_SLOTS  # event: the buffer's previous unit has been reduced and cleared
        self._layer_units = layer_units
        self._install_gather_hooks(layer_units)
        if self.world > 1:
            dist.barrier()

    # -- set-up ------------------------------------------------------------------------------------------
    def _init_shards(self):
        for (so, p0, _n), u in zip(self.pieces, self.units):
            full = max(0, min(u.piece, u.end - p0))
            if full > 0:
                self.master_shard[so:so + full].copy_(self.store.master[p0:p0 + full])
        self.shard.copy_(self.master_shard)

    def _buffer_of(self, u: Unit):
        return self.staging[u.slot] if u.slot >= 0 else self.resident[u.name]

    def _unit_of(self, off: int) -> Unit:
        for u in self.units:
            if u.begin <= off < u.end:
                return u
        raise KeyError(off)

    def _point_views(self):
        """``param.work`` -> staging buffer, ``param.main_grad`` -> gradient space, matrices get their gather record."""
        store = self.store
        for p, off in zip(store.params, store.offsets):
            u = self._unit_of(off)
            d = off - u.begin
            n = p.numel()
            p.work = self._buffer_of(u)[d:d + n].view(p.shape)
            p.main_grad = self.grad_space[u.grad_base + d:u.grad_base + d + n].view(p.shape)
            fused = (self.fused_gather and u.slot >= 0 and p.dim() == 2 and n >= MIN_FUSED_ELEMS and p.shape[1] % 64 == 0
                     and p.shape[0] % 64 == 0)
            p._fsdp = GatherInfo(self, u, d, n) if fused else None
        self._plan_small_ranges()

    def _plan_small_ranges(self):
        """Per unit: the element ranges that the stand-alone copy brings in (everything without a gather record)."""
        store = self.store
        self._small_ranges = {u.name: [] for u in self.units}
        for p, off in zip(store.params, store.offsets):
            if getattr(p, "_fsdp", None) is not None:
                continue
            u = self._unit_of(off)
            d = off - u.begin
            padded = _round_up(p.numel(), 64)
            r = self._small_ranges[u.name]
            if r and r[-1][1] == d:
                r[-1][1] = d + padded
            else:
                r.append([d, d + padded])
        for u in self.units:
            lim = _round_up(u.length, 8)
            self._small_ranges[u.name] = [(a, min(b, lim)) for a, b in self._small_ranges[u.name] if a < lim]

    def _release_master(self):
        """Drop the full fp32 master buffer; parameters keep their shape through a stride-0 view of one NaN."""
        self._nan = torch.full((1,), float("nan"), dtype=torch.float32, device=self.device)
        for p in self.store.params:
            p.data = self._nan.expand(p.shape)
        self.store.master = None

    def _materialise_master(self):
        store = self.store
        if store.master is None:
            store.master = torch.zeros(store.total, dtype=torch.float32, device=self.device)
        for p, off in zip(store.params, store.offsets):
            p.data = store.master[off:off + p.numel()].view(p.shape)

    def _install_gather_hooks(self, layer_units: List[Unit]):
        order = {u.name: i for i, u in enumerate(layer_units)}

        def fwd_pre(u):
            def hook(_module, _inputs):
                self._need(u, prefetch=self._neighbour(order[u.name], +1))
            return hook

        def bwd_pre(u):
            def hook(_module, _grad_out):
                self._need(u, prefetch=self._neighbour(order[u.name], -1), backward=True)
            return hook

        for u in layer_units:
            u.module.register_forward_pre_hook(fwd_pre(u))
            u.module.register_full_backward_pre_hook(bwd_pre(u))
        self.model.register_forward_pre_hook(lambda _m, _i: self.begin_step())

    def _neighbour(self, i: int, d: int) -> Optional[Unit]:
        j = i + d
        return self._layer_units[j] if 0 <= j < len(self._layer_units) else None

    # -- gathers -----------------------------------------------------------------------------------------
    def _launch_gather(self, u: Unit, ranges, stream):
        buf = self._buffer_of(u)
        with torch.cuda.stream(stream):
            for a, b in ranges:
                ops.ext().fsdp_gather(self.rank, self.shard_ptrs, buf, u.shard_off, u.piece, a, b, self.gather_ctas)
                ops.LAUNCHES[0] += 1

    def begin_step(self):
        """Resident units (embeddings, norms, output projection) are refreshed once per step on the compute stream."""
        ctas, self.gather_ctas = self.gather_ctas, 296      # nothing runs beside these copies: use every SM
        for u in self.units:
            if u.slot < 0:
                self._launch_gather(u, [(0, _round_up(u.length, 8))], torch.cuda.current_stream())
        self.gather_ctas = ctas
        self.slot_unit = [None, None]
        self.slot_stamp = [s + 1 for s in self.slot_stamp]
        # events never cross a step boundary (the streams joined when the last backward pass ended); a captured step
        # must not wait on an event that was recorded outside its capture
        self.slot_ready = [None, None]
        self.gslot_free = [None] * GRAD_SLOTS

    def _take_slot(self, u: Unit, stream_for_small):
        """Staging buffer ``u.slot`` changes hands: small parameters (or, unfused, everything) are copied in."""
        cur = torch.cuda.current_stream()
        self.slot_unit[u.slot] = u.name
        self.slot_stamp[u.slot] += 1
        if self.fused_gather:
            # matrices arrive inside their GEMMs (compute stream, naturally ordered behind the slot's previous readers)
            ranges = [(0, _round_up(u.length, 8))] if self._learning else self._small_ranges[u.name]
            self._launch_gather(u, ranges, cur)
            self.slot_ready[u.slot] = None
        else:
            self.side.wait_stream(cur)        # everything already enqueued may still read the slot's previous contents
            self._launch_gather(u, [(0, _round_up(u.length, 8))], self.side)
            ev = torch.cuda.Event()
            ev.record(self.side)
            self.slot_ready[u.slot] = ev

    def _need(self, u: Unit, prefetch: Optional[Unit] = None, backward: bool = False):
        if self.slot_unit[u.slot] != u.name:
            self._take_slot(u, None)
        if self.slot_ready[u.slot] is not None:
            torch.cuda.current_stream().wait_event(self.slot_ready[u.slot])
        if backward and u.gslot >= 0 and self.gslot_free[u.gslot] is not None:
            # the rotating gradient buffer must have been reduced and cleared by its previous user
            torch.cuda.current_stream().wait_event(self.gslot_free[u.gslot])
            self.gslot_free[u.gslot] = None
        if (not self.fused_gather and prefetch is not None and self.slot_unit[prefetch.slot] != prefetch.name
                and prefetch.slot != u.slot):
            self._take_slot(prefetch, None)

    def _claim(self, info: GatherInfo):
        u = info.unit
        if self.slot_unit[u.slot] != u.name:
            raise RuntimeError("a weight of %s is used outside the layer's forward / backward call (fully sharded parameters "
                               "are gathered by the layer's hooks)" % u.name)
        if self._learning:
            info.used = True
            return None
        key = (u.name, self.slot_stamp[u.slot])
        if info.valid_key == key:
            return None
        info.valid_key = key
        ctr = self.gather_counters[u.slot]
        return (self.rank, self.shard_ptrs, self.staging[u.slot], u.shard_off, u.piece, info.offset, info.numel, ctr)

    # -- reductions ----------------------------------------------------------------------------------------
    def _grad_range(self, u: Unit):
        # every unit's buffer (rotating or resident) is cleared by its own reduction once all peers have read it
        return u.grad_base + self.rank * u.piece, (u.grad_base, _round_up(u.piece * self.world, 64))

    def _after_reduce(self, u: Unit):
        if u.gslot >= 0:
            ev = torch.cuda.Event()
            ev.record(self.comm)
            self.gslot_free[u.gslot] = ev

    def __call__(self, flat_grad=None):
        out = super().__call__(flat_grad)
        self.gslot_free = [None] * GRAD_SLOTS      # the streams have joined: nothing is pending any more
        return out

    def _master(self):
        return self.master_shard

    def _zero_len(self) -> int:
        return 0                   # every reduce_unit clears its own gradient buffer

    def _finish_learning(self):
        self._learning = False
        for p in self.store.params:
            info = getattr(p, "_fsdp", None)
            if info is not None and not info.used:
                p._fsdp = None
        self._plan_small_ranges()

    def launch(self):
        super().launch()
        if self._learning:
            self._finish_learning()
        self.slot_unit = [None, None]
        self.slot_stamp = [s + 1 for s in self.slot_stamp]

    # -- checkpoints -----------------------------------------------------------------------------------------
    def gather_master(self):
        """Collective: re-materialise the full fp32 master buffer (``param.data``) on every rank from the owners'
        pieces.  ``release_master`` drops it again."""
        self._materialise_master()
        if self.world > 1:
            everyone = [torch.empty_like(self.master_shard) for _ in range(self.world)]
            dist.all_gather(everyone, self.master_shard)
        else:
            everyone = [self.master_shard]
        for r, shard in enumerate(everyone):
            self._shard_to_flat(shard, self.store.master, r)

    def release_master(self):
        self._release_master()

    def load_master(self, flat_master: Optional[torch.Tensor] = None):
        """After ``param.data`` has been (re)loaded into a materialised master buffer: cut the shards again."""
        src = flat_master if flat_master is not None else self.store.master
        for (so, p0, _n), u in zip(self.pieces, self.units):
            full = max(0, min(u.piece, u.end - p0))
            if full > 0:
                self.master_shard[so:so + full].copy_(src[p0:p0 + full])
        self.shard.copy_(self.master_shard)

    # memory accounting, bytes per rank
    def memory_report(self):
        total = self.store.total
        persistent = 2 * self.shard.numel() + 4 * self.master_shard.numel() + 4 * self.reduced.numel() + 8 * self.exp_avg.numel()
        staging = 2 * sum(b.numel() for b in self.staging) + 2 * sum(b.numel() for b in self.resident.values())
        grad_staging = 4 * self.grad_space.numel()
        return {"bf16_shard": 2 * self.shard.numel(), "master_shard": 4 * self.master_shard.numel(),
                "reduced_grad_shard": 4 * self.reduced.numel(), "optimizer_state": 8 * self.exp_avg.numel(),
                "persistent_bytes_per_param": persistent / max(total, 1), "param_staging": staging,
                "grad_staging": grad_staging, "full_master_resident": self.store.master is not None,
                "replicated_bf16_would_be": 2 * total, "replicated_state_would_be": 16 * total}
