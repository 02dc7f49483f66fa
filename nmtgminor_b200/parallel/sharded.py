"""Unit-wise sharded optimiser step over peer-mapped memory: the machinery shared by data parallelism
(``symmetric.FusedAllReduceAdam``) and fully sharded parameters (``fsdp.FullyShardedAdam``).

The flat parameter space is cut into UNITS: every module of ``model.encoder.layers`` / ``model.decoder.layers`` is
one unit, the parameters between them (embeddings, final norms, output projection) are merged into "resident"
units.  Every unit is cut into ``world`` equal pieces and rank r owns piece r of every unit: Adam moments (and the
reduced gradients) exist only for owned pieces, concatenated in "shard order".

Gradient reduction is overlapped with the backward pass.  A backward pre-hook on every layer notices that the
layer ABOVE it has finished its backward pass (all its weight gradients have been enqueued) and launches that
unit's ``reduce_unit`` kernel on a communication stream, behind an event of the compute stream; the kernel sums
the owned piece over all ranks' gradient buffers with peer loads while the compute stream goes on with the
layers below.  What is left when the backward pass ends (the first layer, the resident units) is reduced then, the
streams join, and one ``update_pieces`` launch exchanges the norm partials, clips, applies Adam(W) to the owned
pieces and publishes the refreshed bf16 parameters.  The same sequence is captured into the step's CUDA graph
(the cross-stream dependencies become fork / join edges).

All ranks must launch the units' reductions in the same order, because each waits for all peers' notice of the
same unit.  Hook order is the reverse layer order on every rank as long as no layer is skipped; models with
stochastic depth (``death_rate`` / layer drop) therefore reduce everything after the backward pass, in a fixed
order.

The reference gets the same overlap from DistributedDataParallel's autograd hooks and 25 MB buckets
(onmt/train_utils/mp_trainer.py:381-387) and, fully sharded, from FSDP's post-backward reduce-scatter
(onmt/train_utils/mp_trainer.py:314-341).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops

FLAG_ROWS = 256            # kNmtgFlagRows of csrc/ops_api.h
FLAG_INTS = FLAG_ROWS * 16
PARTIAL_FLOATS = 2 * 16
FIRST_UNIT_ROW = 4         # rows 0-2: step barriers; unit i uses rows FIRST_UNIT_ROW + 2 i (+1)
MAX_UNITS = 96
PIECE_ALIGN = 64           # elements: a 128-byte row segment of a bf16 matrix never straddles two owners


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class Unit:
    def __init__(self, name: str, begin: int, end: int, module=None):
        self.name, self.begin, self.end, self.module = name, begin, end, module
        self.index = -1
        self.piece = 0          # elements per rank (multiple of PIECE_ALIGN)
        self.shard_off = 0      # offset of this unit's piece in shard-ordered buffers
        self.slot = -1          # parameter staging buffer (0 / 1) or -1 for a resident unit (fully sharded mode)
        self.gslot = -1         # rotating gradient buffer, or -1
        self.grad_base = 0      # offset of the unit's gradients in the gradient space

    @property
    def length(self):
        return self.end - self.begin

    @property
    def row(self):
        return FIRST_UNIT_ROW + 2 * self.index


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
            if any(not store.params[i].requires_grad for i in ids) and any(store.params[i].requires_grad for i in ids):
                continue              # partly frozen layer: its parameters are not contiguous in the flat space
            for i in ids:
                claimed[i] = True
            begin = store.offsets[ids[0]]
            end = store.offsets[ids[-1] + 1] if ids[-1] + 1 < len(store.offsets) else store.total
            layer_units.append(Unit("%s.layers.%d" % (stack_name, li), begin, end, layer))
    layer_units.sort(key=lambda u: u.begin)
    if len(layer_units) > MAX_UNITS - 8:      # very deep stacks: merge neighbouring layers is not needed so far
        layer_units = layer_units[:MAX_UNITS - 8]
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
    for i, u in enumerate(units):
        u.index = i
        u.piece = _round_up(-(-u.length // world), PIECE_ALIGN)
        u.shard_off = off
        off += u.piece
        u.grad_base = u.begin
        if u.module is not None:
            u.slot = n_layer % 2
            n_layer += 1
    assert len(units) <= MAX_UNITS, "too many units"
    return units


def skips_layers(opt) -> bool:
    """True when the model may skip layers at random (every rank then runs a different set of layer hooks)."""
    return any(float(getattr(opt, name, 0) or 0) > 0 for name in ("death_rate", "enc_layerdrop", "dec_layerdrop", "layerdrop",
                                                                  "enc_stochastic_depth", "dec_stochastic_depth"))


class UnitShardedStep:
    """Owned pieces, per-unit reductions overlapped with backward, sharded Adam(W).  Subclasses set ``mode`` (0: bf16
    parameters replicated and refreshed by peer stores, 1: bf16 parameters sharded) and provide the gradient space."""

    fused_optimizer = True
    mode = 0

    def _setup(self, model, store, optim, heap, grad_ptrs, work_ptrs, units: List[Unit], overlap: bool = True):
        self.model, self.store, self.optim, self.heap = model, store, optim, heap
        self.rank, self.world = heap.rank, heap.world
        self.units = units
        dev = store.device
        self.device = dev
        self.shard_len = sum(u.piece for u in units)
        self.flags, self.flag_ptrs = heap.alloc(FLAG_INTS, torch.int32)
        self.partials, self.partial_ptrs = heap.alloc(PARTIAL_FLOATS, torch.float32)
        self.grad_ptrs, self.work_ptrs = grad_ptrs, work_ptrs
        f32 = dict(dtype=torch.float32, device=dev)
        self.reduced = torch.zeros(self.shard_len, **f32)
        self.exp_avg = torch.zeros(self.shard_len, **f32)
        self.exp_avg_sq = torch.zeros(self.shard_len, **f32)
        self.sq = torch.zeros(1, **f32)
        self.nonfinite = torch.zeros(1, dtype=torch.int32, device=dev)
        self.norm = torch.zeros(1, **f32)
        self.epoch = torch.ones(1, dtype=torch.int32, device=dev)
        self.counters = torch.zeros(len(units), dtype=torch.int32, device=dev)
        # this rank's piece of every unit: (offset in shard order, offset in the flat parameter space, length); only the
        # trainable prefix of the flat space is ever updated
        limit = int(getattr(store, "trainable_total", store.total))
        self.pieces = []
        for u in units:
            p0 = u.begin + self.rank * u.piece
            n = max(0, min(u.piece, min(u.end, limit) - p0))
            n -= n % 4
            self.pieces.append((u.shard_off, p0, n))
        # high priority: a reduction's small CTAs are placed as soon as an SM has room, ahead of queued GEMM CTAs
        self.comm = torch.cuda.Stream(device=dev, priority=-1)
        # CTAs (of 128 threads) of a reduction that runs beside the backward pass, and of one that runs after it
        self.reduce_ctas = int(os.environ.get("NMTG_REDUCE_CTAS", "1184"))
        self.tail_ctas = int(os.environ.get("NMTG_REDUCE_TAIL_CTAS", "1184"))
        self.overlap = bool(overlap) and os.environ.get("NMTG_OVERLAP_REDUCE", "1") != "0"
        reserve = int(os.environ.get("NMTG_GEMM_SM_RESERVE", "0"))
        if reserve > 0 and self.overlap and self.world > 1:
            ops.ext().set_gemm_variant(60 + reserve)     # persistent GEMMs leave these SMs to the reductions
        # NMTG_COMM_SMS = n: n SMs are left free by EVERY kernel of the library and the per-layer reductions run there as n
        # wide CTAs (they cannot share an SM with a GEMM or attention CTA), so the reduce-scatter proceeds under the backward
        # pass without slowing the statically scheduled persistent kernels.  The reduction after backward uses the whole GPU.
        self.comm_sms = int(os.environ.get("NMTG_COMM_SMS", "0")) & ~1
        if self.comm_sms > 0 and self.overlap and self.world > 1:
            ops.ext().set_sm_reserve(self.comm_sms)
            self.reduce_ctas = -self.comm_sms
        self.active = True          # hooks launch reductions only during a backward pass that ends in an update
        self._done = set()          # units reduced in the current backward pass
        self._last = None           # layer unit whose backward pass is running
        self._micro = 0             # micro-batches reduced since the last update (fully sharded accumulation)
        self._forked = False
        self._install_reduce_hooks()

    # -- hooks ---------------------------------------------------------------------------------------------
    def _install_reduce_hooks(self):
        def bwd_pre(u):
            def hook(_module, _grad_out):
                self._backward_reaches(u)
            return hook
        for u in self.units:
            if u.module is not None:
                u.module.register_full_backward_pre_hook(bwd_pre(u))

    def _backward_reaches(self, u: Unit):
        """The backward pass is about to enter layer ``u``: the layer it has just left is complete."""
        prev, self._last = self._last, u
        if prev is not None and prev is not u and self.active and self.overlap:
            self._reduce(prev)

    # -- reductions ------------------------------------------------------------------------------------------
    def _grad_range(self, u: Unit):
        """(offset of this rank's piece in the gradient space, range to clear afterwards or (0, 0))."""
        return u.grad_base + self.rank * u.piece, (0, 0)

    def _reduce(self, u: Unit, tail: bool = False):
        if u.index in self._done:
            return
        self._done.add(u.index)
        so, p0, n = self.pieces[u.index]
        cur = torch.cuda.current_stream()
        self.comm.wait_stream(cur)               # every weight gradient of the unit has been enqueued before this point
        self._forked = True
        g0, (zb, zl) = self._grad_range(u)
        with torch.cuda.stream(self.comm):
            ops.ext().reduce_unit(self.rank, self.grad_ptrs, self.flag_ptrs, u.row, self.reduced[so:so + max(n, 4)], g0, n,
                                  self._micro > 0 and self.mode == 1, zb, zl, self.counters[u.index:u.index + 1], self.epoch,
                                  self.tail_ctas if tail else self.reduce_ctas)
            self._after_reduce(u)
        ops.LAUNCHES[0] += 1

    def _after_reduce(self, u: Unit):
        pass

    def __call__(self, flat_grad=None):
        """End of a backward pass: reduce whatever the hooks have not, in a fixed order, and join the streams."""
        if not self.active:
            self._last = None
            return None
        for u in reversed(self.units):
            self._reduce(u, tail=True)       # nothing left to overlap with: use the whole GPU
        if self._forked:
            torch.cuda.current_stream().wait_stream(self.comm)
            self._forked = False
        self._done = set()
        self._last = None
        self._micro += 1
        return None

    # -- optimiser interface -------------------------------------------------------------------------------
    def _master(self):
        return self.store.master

    def _zero_len(self) -> int:
        return self.store.total

    def launch(self):
        e = ops.ext()
        self.sq.zero_()
        self.nonfinite.zero_()
        e.sq_norm(self.reduced, self.sq, self.nonfinite)
        e.update_pieces(self.rank, self.grad_ptrs, self.work_ptrs, self.flag_ptrs, self.partial_ptrs, [p[0] for p in self.pieces],
                        [p[1] for p in self.pieces], [p[2] for p in self.pieces], self.reduced, self._master(), self.exp_avg,
                        self.exp_avg_sq, self.optim.hyper, self.sq, self.nonfinite, self.mode, self._zero_len(), self.epoch,
                        self.norm)
        e.peer_finish_step(self.rank, self.flag_ptrs, self.epoch)
        ops.LAUNCHES[0] += 2
        self._micro = 0

    # -- optimiser state in the flat layout (checkpoints are independent of the world size) -------------------
    def _shard_to_flat(self, shard: torch.Tensor, flat: torch.Tensor, rank: int):
        for u in self.units:
            p0 = u.begin + rank * u.piece
            n = max(0, min(u.piece, u.end - p0))
            if n > 0:
                flat[p0:p0 + n].copy_(shard[u.shard_off:u.shard_off + n])

    def _flat_to_shard(self, flat: torch.Tensor, shard: torch.Tensor):
        shard.zero_()
        for u in self.units:
            p0 = u.begin + self.rank * u.piece
            n = max(0, min(u.piece, min(u.end, flat.numel()) - p0))
            if n > 0:
                shard[u.shard_off:u.shard_off + n].copy_(flat[p0:p0 + n])

    def gather_flat(self, shard: torch.Tensor, to_cpu: bool = True) -> Optional[torch.Tensor]:
        """Collective: the shard-ordered fp32 buffers of all ranks -> one flat-ordered tensor on rank 0 (None elsewhere)."""
        if self.world > 1:
            everyone = [torch.empty_like(shard) for _ in range(self.world)] if self.rank == 0 else None
            dist.gather(shard, everyone, dst=0)
        else:
            everyone = [shard]
        if self.rank != 0:
            return None
        flat = torch.zeros(self.store.total, dtype=shard.dtype, device="cpu" if to_cpu else shard.device)
        for r, s in enumerate(everyone):
            self._shard_to_flat(s.cpu() if to_cpu else s, flat, r)
        return flat

    def gather_moments(self):
        """Collective (every rank must call it): flat-ordered Adam moments on rank 0."""
        m = self.gather_flat(self.exp_avg)
        v = self.gather_flat(self.exp_avg_sq)
        return (m, v) if self.rank == 0 else None

    def load_moments(self, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor):
        """Flat-ordered moments (any world size wrote them) -> this rank's pieces."""
        self._flat_to_shard(exp_avg.to(self.device, torch.float32), self.exp_avg)
        self._flat_to_shard(exp_avg_sq.to(self.device, torch.float32), self.exp_avg_sq)

    def state_dict(self):
        raise RuntimeError("sharded optimiser state is saved through gather_moments(), which every rank has to call")
