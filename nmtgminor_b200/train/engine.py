"""Training-step engine: host batch in, loss out, everything in between enqueued on one CUDA stream.

One ``TrainEngine.train_step(batch)`` call performs: async host-to-device copy of the packed integer
tensors from pinned memory, forward through the fused kernels, backward (weight gradients accumulate
straight into the flat fp32 buffer), optional data-parallel reduction of that buffer, and the flat
Adam(W) update.  With ``cuda_graph=True`` forward + backward + update are captured into a CUDA graph once per SHAPE CLASS
of batches (packed capacities rounded to a few sizes) and replayed per step (inputs are copied into static
buffers, per-step scalars live in device memory, dropout masks advance through a device-resident seed
word), which removes per-kernel launch and Python overhead from the step.

The reference's equivalent loop is ``Trainer.train_epoch`` (onmt/train_utils/mp_trainer.py:743-1016):
``Batch.cuda`` -> autocast forward -> loss -> ``GradScaler.scale(loss).backward()`` (DDP all-reduce inside)
-> unscale / normalise / clip -> ``optim.step`` -> ``zero_grad``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..models.layers import PackedSeqs
from ..parallel.flat import FlatParameterStore
from .optim import Optim


class _StaticInputs:
    """Device buffers with fixed addresses that a captured graph reads its batch from."""

    def __init__(self, batch, device):
        src, tgt = batch.packed_source(), batch.packed_target_input()
        mk = lambda t: torch.empty_like(t, device=device)
        self.src = PackedSeqs(mk(src.tokens), mk(src.positions), mk(src.cu), src.max_len)
        self.tgt = PackedSeqs(mk(tgt.tokens), mk(tgt.positions), mk(tgt.cu), tgt.max_len)
        self.labels = mk(batch.packed_target_output())

    def signature(self):
        return (self.src.tokens.numel(), self.src.cu.numel(), self.src.max_len, self.tgt.tokens.numel(),
                self.tgt.cu.numel(), self.tgt.max_len)

    @staticmethod
    def signature_of(batch):
        s, t = batch.packed_source(), batch.packed_target_input()
        return (s.tokens.numel(), s.cu.numel(), s.max_len, t.tokens.numel(), t.cu.numel(), t.max_len)

    def load(self, batch):
        s, t = batch.packed_source(), batch.packed_target_input()
        self.src.tokens.copy_(s.tokens, non_blocking=True)
        self.src.positions.copy_(s.positions, non_blocking=True)
        self.src.cu.copy_(s.cu, non_blocking=True)
        self.tgt.tokens.copy_(t.tokens, non_blocking=True)
        self.tgt.positions.copy_(t.positions, non_blocking=True)
        self.tgt.cu.copy_(t.cu, non_blocking=True)
        self.labels.copy_(batch.packed_target_output(), non_blocking=True)

    # Batch protocol used by the models
    def packed_source(self):
        return self.src

    def packed_target_input(self):
        return self.tgt

    def packed_target_output(self):
        return self.labels


class TrainEngine:
    def __init__(self, model: torch.nn.Module, opt, device=None, reducer=None, cuda_graph: bool = False,
                 grad_scale: float = 1.0, ddp: Optional[str] = None):
        """``ddp``: None (single process or an explicit ``reducer`` callable), ``"nccl"`` (all-reduce of the flat
        gradient buffer through torch.distributed) or ``"fused"`` (peer-memory reduce-scatter + sharded Adam(W) +
        all-gather kernels; needs an initialised process group on one node)."""
        self.model = model
        self.opt = opt
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.on_gpu = self.device.type == "cuda"
        import torch.distributed as dist
        world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        self.world_size = world
        heap = None
        ptrs = {}
        fsdp = ddp == "fsdp" and self.on_gpu and ops.extension_available()
        if (fsdp or (ddp == "fused" and world > 1)) and self.on_gpu and ops.extension_available():
            from ..parallel.symmetric import SymmetricHeap
            heap = SymmetricHeap(self.device)

            def symm(name):
                def alloc(n, dt):
                    t, p = heap.alloc(n, dt)
                    ptrs[name] = p
                    return t
                return alloc
            # fully sharded: no replicated bf16 copy and no full gradient buffer; layers read gathered weights from
            # staging buffers and write gradients into rotating per-layer buffers owned by the sharded step
            nothing = lambda n, dt: None
            self.store = FlatParameterStore(model, self.device, pad_total_to=256 * world,
                                            allocator={"grad": nothing if fsdp else symm("grad"), "work": nothing if fsdp else symm("work")})
        else:
            self.store = FlatParameterStore(model, self.device, pad_total_to=256 * max(world, 1))
        for b in model.buffers():
            b.data = b.data.to(self.device)
        self.optim = Optim(opt)
        self.optim.set_parameters(model.parameters(), self.store, allocate_state=heap is None)
        from ..parallel.sharded import skips_layers
        overlap = not skips_layers(opt)
        if fsdp:
            from ..parallel.ddp import broadcast_parameters
            from ..parallel.fsdp import FullyShardedAdam
            if world > 1:
                broadcast_parameters(self.store)
            assert self.optim.fused, "-fsdp needs the fused Adam(W) path"
            reducer = FullyShardedAdam(model, self.store, self.optim, heap, overlap=overlap)
            self.optim.attach_distributed(reducer)
        elif world > 1 and reducer is None and ddp is not None:
            from ..parallel.ddp import NcclReducer, broadcast_parameters
            broadcast_parameters(self.store)
            if heap is not None and self.optim.fused:
                from ..parallel.symmetric import FusedAllReduceAdam
                reducer = FusedAllReduceAdam(self.store, self.optim, heap, ptrs["grad"], ptrs["work"], model=model, overlap=overlap)
                self.optim.attach_distributed(reducer)
            else:
                if heap is not None:     # the fused path was planned but the optimiser is not Adam-like
                    self.optim.set_parameters(model.parameters(), self.store)
                reducer = NcclReducer(world)
        self.reducer = reducer            # callable(flat_grad) -> None, data-parallel gradient reduction
        self.grad_scale = grad_scale
        self.loss_weight = 1.0            # weight of the next batch's gradient (replay weighting in continual learning)
        # -fp16 without -bf16: the fp16 protocol (dynamic loss scale, skipped steps) on the bf16 kernels; the scale lives
        # on the device, so the captured step carries it
        self.scaler = None
        from .loss_scaler import DynamicLossScaler, wants_loss_scaling
        if wants_loss_scaling(opt):
            self.scaler = DynamicLossScaler(self.device, init_scale=float(getattr(opt, "init_loss_scale", 2.0 ** 16) or 2.0 ** 16),
                                            growth_interval=int(getattr(opt, "loss_scale_window", 2000) or 2000))
            self.optim.loss_scaler = self.scaler
        # only models that declare it: a captured step sees nothing of a batch but its packed token views
        self.use_graph = bool(cuda_graph) and self.on_gpu and bool(getattr(model, "graph_capturable", False))
        self._graphs = {}                 # shape class -> [graph, static inputs, launches per replay, last use]
        self._seen = {}                   # shape class -> batches met so far (a class is captured at batch number capture_after)
        self._pool = None
        self._tick = 0
        self.max_graphs = 64
        self.capture_after = 1            # trainers that stream a token-budget data set raise this (rare classes stay eager)
        self.evict_graphs = True          # False: once the cache is full, further classes run kernel by kernel for good
        self.kernel_launches_per_step = 0

    # ---------------------------------------------------------------------------------------------
    def _forward_backward(self, batch):
        from ..utils.tracing import nvtx_range
        trace = bool(getattr(self.opt, "trace_nvtx", False))
        if trace and not getattr(self, "_nvtx_hooks", None):
            from ..utils.tracing import install_nvtx_hooks
            self._nvtx_hooks = install_nvtx_hooks(self.model)
        ops.reset_stream_counter()
        if hasattr(self.model, "num_updates"):
            self.model.num_updates = int(self.optim._step)      # schedules inside the model (delayed CTC weight)
        # the loss gradient is written pre-scaled by the kernel (scale 1): no [tokens, V] rescale pass in backward
        with nvtx_range("forward", trace):
            weight = float(getattr(self, "loss_weight", 1.0))       # per-step weight of this batch's gradient
            gs = weight if self.scaler is None else (self.scaler.scale if weight == 1.0 else self.scaler.scale * weight)
            out = self.model(batch, grad_scale=gs)
        with nvtx_range("backward", trace):
            out["loss"].backward()
        if not self.optim.fused:
            pass
        else:
            self.store.gather_autograd_grads()   # parameters touched by unfused ops, if any
        return out["loss"].detach(), out["correct"].detach()

    def _eager_step(self, batch, update: bool = True):
        if self.on_gpu:
            batch = batch.cuda(self.device, hot_only=True)
            if ops.extension_available():
                # dropout masks are a function of (seed + device seed word, op index, element): a new word per call gives
                # every step and every accumulation micro-batch its own masks (a captured graph does the same inside)
                ops.advance_device_seed(self.device.index)
        n0 = ops.LAUNCHES[0]
        if hasattr(self.reducer, "active"):
            # data parallel: micro-batches that do not end in an update accumulate locally, nothing is exchanged
            self.reducer.active = update or getattr(self.reducer, "mode", 0) == 1
        loss, correct = self._forward_backward(batch)
        if not update and hasattr(self.reducer, "active") and self.reducer.active:
            self.reducer(self.store.grad)       # fully sharded: every micro-batch is reduce-scattered into the shard
        if update:
            from ..utils.tracing import nvtx_range
            with nvtx_range("reduce+optimizer", bool(getattr(self.opt, "trace_nvtx", False))):
                if self.reducer is not None and not self.optim.fused:
                    # torch.optim path (CPU / gloo ranks, optimisers without a flat kernel): autograd left the gradients
                    # in p.grad; move them into the flat buffer, reduce that, and hand the optimiser views of it
                    self.store.gather_autograd_grads()
                    self.reducer(self.store.grad)
                    for p in self.store.params:
                        if p.requires_grad:
                            p.grad = p.main_grad
                elif self.reducer is not None:
                    self.reducer(self.store.grad)
                self.optim.step(self.grad_scale)
            if not self.optim.fused:
                self.optim.zero_grad()
        self.kernel_launches_per_step = ops.LAUNCHES[0] - n0
        if update:
            self._snapshot_status()
        return loss, correct

    def _snapshot_status(self):
        """Copies the device status word into pinned host memory behind the step (asynchronous; inside a capture it
        becomes a node of the graph), so ``peek_status`` sees a timed-out wait one step later without synchronising."""
        if not (self.on_gpu and self.world_size > 1 and ops.extension_available()):
            return
        if getattr(self, "_status_host", None) is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_host.copy_(ops.ext().get_status_tensor(self.device.index), non_blocking=True)

    def peek_status(self) -> int:
        """Status word as of the last completed step (no device synchronisation); 0 = every wait was answered."""
        h = getattr(self, "_status_host", None)
        return int(h[0]) if h is not None else 0

    def local_only_mode(self):
        """Measurement aid: from now on every rank updates its own full parameter copy from its own gradients (gradient
        norm + flat Adam(W), what a single GPU does) and nothing is exchanged.  The difference between a step before and
        after this call is the part of the gradient exchange that the backward pass did not hide.  The ranks' parameters
        diverge afterwards, so this is the last thing a benchmark does with the engine."""
        if getattr(self.optim, "distributed", None) is None or getattr(self.reducer, "mode", 0) != 0:
            return
        torch.cuda.synchronize()
        self._graphs = {}
        self.reducer.active = False        # its backward hooks stay installed on the layers
        self.reducer.overlap = False
        self.reducer = None
        self.optim.distributed = None
        n = self.optim.n_update
        self.optim.exp_avg = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.optim.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.store.zero_grad()

    def _capture(self, batch, sig):
        """Capture forward + backward + reduction + update for batches of this shape class.  Nothing is executed here:
        the caller has just run the same step eagerly (which also warmed the allocator pools, the tensor-map cache and
        every lazy initialisation), and with several ranks a capture must not add or remove a step from the sequence of
        collective steps that the peers see."""
        static = _StaticInputs(batch, self.device)
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()     # all shape classes share one private memory pool
            self._loss_out = torch.zeros(1, dtype=torch.float32, device=self.device)
            self._correct_out = torch.zeros(1, dtype=torch.float32, device=self.device)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = ops.LAUNCHES[0]
        step_before = self.optim._step
        # thread-local capture mode: the data loader's worker / pinning threads keep allocating pinned host memory while
        # this thread captures, which a global-mode capture treats as an error
        with torch.cuda.graph(graph, pool=self._pool, capture_error_mode="thread_local"):
            ops.advance_device_seed(self.device.index)
            loss, correct = self._forward_backward(static)
            if self.reducer is not None:
                self.reducer(self.store.grad)
            self.optim.launch_fused()
            self._snapshot_status()
            # results leave the pool: the next replay (of any shape class) may reuse the pool's memory
            self._loss_out.copy_(loss.reshape(1))
            self._correct_out.copy_(correct.reshape(1).float())
        self.optim._step = step_before
        launches = ops.LAUNCHES[0] - n0               # every replay re-runs exactly these launches
        if len(self._graphs) >= self.max_graphs:      # drop the least recently used shape class
            oldest = min(self._graphs, key=lambda k: self._graphs[k][3])
            del self._graphs[oldest]
        self._graphs[sig] = [graph, static, launches, self._tick]
        return self._graphs[sig]

    def train_step(self, batch, update: bool = True):
        """Forward + backward on ``batch`` (host tensors, ideally pinned) and, when ``update`` is set, gradient
        reduction + one optimiser update (``update=False`` only accumulates gradients).  Returns (loss_sum,
        n_correct) as 1-element device tensors; reading them is the only synchronisation point.

        With ``cuda_graph`` the first batch of every shape class (packed capacities, sentence count, length bounds: see
        ``data.dataset.bucket_capacity``) runs kernel by kernel and is then captured; later batches of the class replay
        the graph.  The returned tensors are overwritten by the next step."""
        self.model.train()
        if not (self.use_graph and self.optim.fused) or not update:
            return self._eager_step(batch, update)
        if hasattr(self.reducer, "active"):
            self.reducer.active = True
        self._tick += 1
        sig = _StaticInputs.signature_of(batch)
        entry = self._graphs.get(sig)
        if entry is None:
            # a capture costs several eager steps (a second pass over the step's launches plus the instantiation of a
            # graph of a few hundred nodes): classes that a token-budget data set produces once or twice run eagerly
            seen = self._seen.get(sig, 0) + 1
            self._seen[sig] = seen
            out = self._eager_step(batch, True)
            if seen >= self.capture_after and (self.evict_graphs or len(self._graphs) < self.max_graphs):
                self._capture(batch, sig)
            return out
        graph, static, launches, _ = entry
        entry[3] = self._tick
        static.load(batch)
        self.optim._step += 1
        self.optim.write_hyper(self.grad_scale)
        graph.replay()
        self.kernel_launches_per_step = launches
        return self._loss_out, self._correct_out

    @torch.no_grad()
    def eval_step(self, batch):
        self.model.eval()
        if self.on_gpu:
            batch = batch.cuda(self.device, hot_only=True)
        out = self.model(batch)
        return out["loss"], out["correct"]
