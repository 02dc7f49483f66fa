"""Fully sharded data parallelism (``-fsdp``) over peer-mapped memory on one NVSwitch node.

Parameters are grouped into UNITS: every module of ``model.encoder.layers`` / ``model.decoder.layers`` is one unit,
everything else (embeddings, final norms, output projection) forms the resident unit.  Rank r keeps piece r of every
unit: bf16 parameters (in the symmetric heap, where peers read them), fp32 master weights and Adam moments.  Full
bf16 weights of a layer exist only while the layer needs them, in one of two staging buffers:

* forward: a pre-forward hook on layer i makes the compute stream wait for the gather of unit i and enqueues the
  gather of unit i + 1 into the other buffer on a side stream, so the peer loads overlap layer i's GEMMs;
* backward: a pre-backward hook does the same in reverse order (the weights are gathered again rather than kept);
* after backward one launch sequence reduce-scatters the gradients straight into shard order, applies Adam(W) to the
  shard and refreshes the bf16 shard that the next step's gathers read (``ops.ext().fsdp_step``).

The gather kernels need no flags (shards only change inside the step barrier); every cross-GPU wait is bounded and
reports through the status word.  The fp32 master copy that backs ``param.data`` stays full-size on every rank for
checkpointing and is refreshed by ``gather_master``; gradients are accumulated full-size and reduced once per step.

Reference behaviour: FSDP wrapping of the encoder / decoder layers, onmt/train_utils/mp_trainer.py:330-350.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops
from .symmetric import FLAG_INTS, PARTIAL_FLOATS, SymmetricHeap


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class Unit:
    def __init__(self, name: str, begin: int, end: int, module=None):
        self.name, self.begin, self.end, self.module = name, begin, end, module
        self.piece = 0          # elements per rank (multiple of 8)
        self.shard_off = 0      # offset of this unit's piece in shard-ordered buffers
        self.slot = -1          # staging buffer (0 / 1) or -1 for the resident unit

    @property
    def length(self):
        return self.end - self.begin


def plan_units(model, store, world: int) -> List[Unit]:
    """Contiguous flat ranges: one per encoder / decoder layer, the rest merged into resident units."""
    index = {id(p): i for i, p in enumerate(store.params)}
    claimed = {}
    layer_units = []
    for stack_name in ("encoder", "decoder"):
        stack = getattr(model, stack_name, None)
        layers = getattr(stack, "layers", None)
        if layers is None:
            continue
        for li, layer in enumerate(layers):
            ids = sorted(index[id(p)] for p in layer.parameters() if id(p) in index and index[id(p)] not in claimed)
            if not ids or ids != list(range(ids[0], ids[-1] + 1)):
                continue              # parameters shared with other modules or not contiguous: leave them resident
            for i in ids:
                claimed[i] = True
            begin = store.offsets[ids[0]]
            end = store.offsets[ids[-1] + 1] if ids[-1] + 1 < len(store.offsets) else store.total
            layer_units.append(Unit("%s.layers.%d" % (stack_name, li), begin, end, layer))
    layer_units.sort(key=lambda u: u.begin)
    units: List[Unit] = []
    cursor = 0
    for u in layer_units:
        if u.begin > cursor:
            units.append(Unit("resident%d" % len(units), cursor, u.begin))
        units.append(u)
        cursor = u.end
    if cursor < store.total:
        units.append(Unit("resident%d" % len(units), cursor, store.total))
    off = 0
    n_layer = 0
    for u in units:
        u.piece = _round_up(-(-u.length // world), 8)
        u.shard_off = off
        off += u.piece
        if u.module is not None:
            u.slot = n_layer % 2
            n_layer += 1
    return units


class FullyShardedAdam:
    """Sharded parameters + optimiser state with gather-on-demand staging; plugs into ``Optim.attach_distributed``."""

    fused_optimizer = True

    def __init__(self, model, store, optim, heap: SymmetricHeap, grad_ptrs, gather_ctas: int = 32):
        assert store.work is None, "the flat store must be built without a full bf16 copy"
        self.model, self.store, self.optim, self.heap = model, store, optim, heap
        self.rank, self.world = heap.rank, heap.world
        dev = store.master.device
        self.units = plan_units(model, store, self.world)
        assert len(self.units) <= 96, "too many units"
        self.shard_len = sum(u.piece for u in self.units)
        self.gather_ctas = gather_ctas
        # symmetric buffers: bf16 shard (peers read it), flags, norm partials
        self.shard, self.shard_ptrs = heap.alloc(self.shard_len, torch.bfloat16)
        self.flags, self.flag_ptrs = heap.alloc(FLAG_INTS, torch.int32)
        self.partials, self.partial_ptrs = heap.alloc(PARTIAL_FLOATS, torch.float32)
        self.grad_ptrs = grad_ptrs
        f32 = dict(dtype=torch.float32, device=dev)
        self.master_shard = torch.zeros(self.shard_len, **f32)
        self.exp_avg = torch.zeros(self.shard_len, **f32)
        self.exp_avg_sq = torch.zeros(self.shard_len, **f32)
        self.reduced = torch.zeros(self.shard_len, **f32)
        self.sq = torch.zeros(1, **f32)
        self.nonfinite = torch.zeros(1, dtype=torch.int32, device=dev)
        self.norm = torch.zeros(1, **f32)
        self.epoch = torch.ones(1, dtype=torch.int32, device=dev)
        # this rank's piece of every unit, in the flat space
        self.pieces = []
        for u in self.units:
            g0 = u.begin + self.rank * u.piece
            n = max(0, min(u.piece, u.end - g0))
            n -= n % 4
            self.pieces.append((u.shard_off, g0, n))
        self._init_shards()
        # staging: two rotating buffers for layer units, one persistent buffer per resident unit
        layer_units = [u for u in self.units if u.slot >= 0]
        max_len = max([u.piece * self.world for u in layer_units], default=8)
        self.staging = [torch.zeros(max_len, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.resident = {u.name: torch.zeros(u.piece * self.world, dtype=torch.bfloat16, device=dev) for u in self.units if u.slot < 0}
        self._point_work_views()
        self.side = torch.cuda.Stream(device=dev)
        self.slot_unit = [None, None]          # which unit each staging buffer holds (or is being filled with)
        self.slot_ready = [None, None]         # event: gather into the slot finished
        self._install_hooks(layer_units)
        if self.world > 1:
            dist.barrier()

    # -- set-up ------------------------------------------------------------------------------------------
    def _init_shards(self):
        for (so, g0, n) in self.pieces:
            if n > 0:
                self.master_shard[so:so + n].copy_(self.store.master[g0:g0 + n])
        self.shard.copy_(self.master_shard)

    def _buffer_of(self, u: Unit):
        return self.staging[u.slot] if u.slot >= 0 else self.resident[u.name]

    def _point_work_views(self):
        store = self.store
        bounds = [(u.begin, u.end, u) for u in self.units]
        for p, off in zip(store.params, store.offsets):
            for b, e, u in bounds:
                if b <= off < e:
                    p.work = self._buffer_of(u)[off - b:off - b + p.numel()].view(p.shape)
                    break

    def _install_hooks(self, layer_units: List[Unit]):
        order = {u.name: i for i, u in enumerate(layer_units)}
        self._layer_units = layer_units

        def fwd_pre(u):
            def hook(_module, _inputs):
                self._need(u, prefetch=self._neighbour(order[u.name], +1))
            return hook

        def bwd_pre(u):
            def hook(_module, _grad_out):
                self._need(u, prefetch=self._neighbour(order[u.name], -1))
            return hook

        for u in layer_units:
            u.module.register_forward_pre_hook(fwd_pre(u))
            u.module.register_full_backward_pre_hook(bwd_pre(u))
        self.model.register_forward_pre_hook(lambda _m, _i: self.begin_step())

    def _neighbour(self, i: int, d: int) -> Optional[Unit]:
        j = i + d
        return self._layer_units[j] if 0 <= j < len(self._layer_units) else None

    # -- gathers -----------------------------------------------------------------------------------------
    def _launch_gather(self, u: Unit, stream):
        with torch.cuda.stream(stream):
            ops.ext().fsdp_gather(self.rank, self.shard_ptrs, self._buffer_of(u), u.shard_off, u.piece, min(u.piece * self.world, _round_up(u.length, 8)),
                                  self.gather_ctas)
        ops.LAUNCHES[0] += 1

    def begin_step(self):
        """Resident units (embeddings, norms, output projection) are refreshed once per step on the compute stream."""
        for u in self.units:
            if u.slot < 0:
                self._launch_gather(u, torch.cuda.current_stream())
        self.slot_unit = [None, None]

    def _gather_into_slot(self, u: Unit):
        cur = torch.cuda.current_stream()
        # everything already enqueued on the compute stream may still read the slot's previous contents
        self.side.wait_stream(cur)
        self._launch_gather(u, self.side)
        ev = torch.cuda.Event()
        ev.record(self.side)
        self.slot_unit[u.slot], self.slot_ready[u.slot] = u.name, ev

    def _need(self, u: Unit, prefetch: Optional[Unit] = None):
        if self.slot_unit[u.slot] != u.name:
            self._gather_into_slot(u)
        torch.cuda.current_stream().wait_event(self.slot_ready[u.slot])
        if prefetch is not None and self.slot_unit[prefetch.slot] != prefetch.name and prefetch.slot != u.slot:
            self._gather_into_slot(prefetch)

    # -- optimiser interface -------------------------------------------------------------------------------
    def __call__(self, flat_grad):
        return None

    def launch(self):
        s = self.store
        ops.ext().fsdp_step(self.rank, self.grad_ptrs, self.shard_ptrs, self.flag_ptrs, self.partial_ptrs,
                            [p[0] for p in self.pieces], [p[1] for p in self.pieces], [p[2] for p in self.pieces], self.reduced,
                            self.sq, self.nonfinite, self.master_shard, self.exp_avg, self.exp_avg_sq, self.optim.hyper,
                            self.shard_len, s.total, self.epoch, self.norm)
        ops.LAUNCHES[0] += 3
        self.slot_unit = [None, None]

    def gather_master(self):
        """Refresh the full fp32 master buffer (``param.data``) on every rank from the owners' pieces."""
        if self.world > 1:
            everyone = [torch.empty_like(self.master_shard) for _ in range(self.world)]
            dist.all_gather(everyone, self.master_shard)
        else:
            everyone = [self.master_shard]
        for r, shard in enumerate(everyone):
            for u in self.units:
                g0 = u.begin + r * u.piece
                n = max(0, min(u.piece, u.end - g0))
                if n > 0:
                    self.store.master[g0:g0 + n].copy_(shard[u.shard_off:u.shard_off + n])

    def state_dict(self):
        return {"exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(), "begin": -self.rank - 1, "length": self.shard_len}

    # memory accounting, bytes per rank
    def memory_report(self):
        total = self.store.total
        return {"bf16_shard": 2 * self.shard_len, "staging": 2 * sum(b.numel() for b in self.staging) + 2 * sum(b.numel() for b in self.resident.values()),
                "optimizer_state": 16 * self.shard_len, "replicated_bf16_would_be": 2 * total, "replicated_state_would_be": 16 * total}
