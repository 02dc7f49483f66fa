"""Optimiser wrapper with the reference's update rules and learning-rate schedules.

``Optim`` drives either

* the flat fused path: one squared-norm kernel + one Adam(W) kernel over the ``FlatParameterStore`` buffers
  (unscale, global-norm clipping with the coefficient computed on the device, update of the fp32 master,
  refresh of the bf16 working copy, gradient zeroing), with the per-step scalars uploaded into a small
  device struct so the sequence can sit inside a captured CUDA graph; or
* plain ``torch.optim`` objects (CPU, or models without a flat store).

Rules kept from the reference (onmt/optim.py:294-559): Adam with eps 1e-9 and betas (0.9, 0.997) by
default, AdamW iff ``weight_decay > 0``; schedules ``noam`` (``lr = init * min(step^-0.5, step *
warmup^-1.5)`` with ``init = model_size^-0.5 * learning_rate``), ``noam_nowarmup``, ``noam_half``,
``cosine``, ``regular`` (+ optional ``lr_decay`` per epoch); ``_step`` travels in the state dict.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..parallel.flat import FlatParameterStore


def learning_rate_at(step: int, opt, init_lr: float) -> float:
    """Schedule value for (1-based) update number ``step``."""
    method = getattr(opt, "update_method", "regular")
    warmup = max(1, getattr(opt, "warmup_steps", 4096))
    step = max(1, step)
    if method in ("noam", "gradient_scaling"):
        return init_lr * min(step ** -0.5, step * warmup ** -1.5)
    if method == "noam_nowarmup":
        return init_lr * max(step, warmup) ** -0.5
    if method == "noam_half":
        return init_lr * min(step ** -0.5, step * warmup ** -1.5) * 0.5 if step > warmup else \
            init_lr * step * warmup ** -1.5
    if method == "cosine":
        max_step = max(getattr(opt, "max_step", 0) or getattr(opt, "max_steps", 0) or 100000, warmup + 1)
        if step <= warmup:
            return getattr(opt, "learning_rate", 1.0) * step / warmup
        prog = min(1.0, (step - warmup) / (max_step - warmup))
        base, floor = getattr(opt, "learning_rate", 1.0), getattr(opt, "min_learning_rate", 0.0) if hasattr(opt, "min_learning_rate") else 0.0
        return floor + 0.5 * (base - floor) * (1.0 + math.cos(math.pi * prog))
    return getattr(opt, "learning_rate", 1.0)   # 'regular'


class Optim:
    def __init__(self, opt):
        self.opt = opt
        self.method = getattr(opt, "optim", "adam").lower()
        self.lr = getattr(opt, "learning_rate", 1.0)
        self.update_method = getattr(opt, "update_method", "regular")
        self.model_size = getattr(opt, "model_size", 512)
        if self.update_method in ("noam", "noam_nowarmup", "noam_half", "gradient_scaling"):
            self.init_lr = self.model_size ** -0.5 * self.lr
        else:
            self.init_lr = self.lr
        self.beta1, self.beta2 = getattr(opt, "beta1", 0.9), getattr(opt, "beta2", 0.997)
        self.eps = 1e-9
        self.weight_decay = getattr(opt, "weight_decay", 0.0)
        self.max_grad_norm = getattr(opt, "max_grad_norm", 0.0)
        self.lr_decay = getattr(opt, "learning_rate_decay", 1.0)
        self.start_decay_at = getattr(opt, "start_decay_at", 99999)
        self._step = 0
        if int(getattr(opt, "starting_step", -1) or -1) > 0:
            self._step = int(opt.starting_step)     # -starting_step: continue the schedule of an earlier run
        self._epoch_decay = 1.0
        self.store: Optional[FlatParameterStore] = None
        self.optimizer: Optional[torch.optim.Optimizer] = None
        self.params = []

    # -- attach -----------------------------------------------------------------------------------
    def set_parameters(self, params, store: Optional[FlatParameterStore] = None, allocate_state: bool = True):
        """Fused flat path when ``store`` lives on a CUDA device and the method is Adam-like.  ``allocate_state=False``
        when a sharded step (``attach_distributed``) will own the moments."""
        self.params = [p for p in params if p.requires_grad]
        self.store = store
        # -amsgrad keeps a running maximum of the second moment, which the flat kernel does not: torch.optim handles it
        self.amsgrad = bool(getattr(self.opt, "amsgrad", False))
        fused = (store is not None and store.master.is_cuda and self.method in ("adam", "adamw") and ops.extension_available()
                 and not self.amsgrad)
        self.fused = fused
        if fused:
            dev = store.master.device
            # moments only for the trainable prefix of the flat space (frozen parameters sit behind it)
            self.n_update = int(getattr(store, "trainable_total", store.total))
            self.exp_avg = torch.zeros(self.n_update, dtype=torch.float32, device=dev) if allocate_state else None
            self.exp_avg_sq = torch.zeros(self.n_update, dtype=torch.float32, device=dev) if allocate_state else None
            self.grad_sq = torch.zeros(1, dtype=torch.float32, device=dev)
            self.nonfinite = torch.zeros(1, dtype=torch.int32, device=dev)
            self.hyper = torch.zeros(16, dtype=torch.float32, device=dev)
            self._hyper_host = torch.zeros(16, dtype=torch.float32).pin_memory() if torch.cuda.is_available() else torch.zeros(16)
            return
        if self.method == "sgd":
            self.optimizer = torch.optim.SGD(self.params, lr=self.lr, weight_decay=self.weight_decay, momentum=0.0)
        elif self.method in ("adam", "adamw", "fused_adam"):
            cls = torch.optim.AdamW if self.weight_decay > 0 else torch.optim.Adam
            self.optimizer = cls(self.params, lr=self.lr, betas=(self.beta1, self.beta2), eps=self.eps,
                                 weight_decay=self.weight_decay, amsgrad=self.amsgrad)
        elif self.method == "adafactor":
            from .adafactor import Adafactor
            self.optimizer = Adafactor(self.params, lr=self.lr if self.lr < 1 else None, weight_decay=self.weight_decay)
        elif self.method == "lion":
            from .lion import Lion
            self.optimizer = Lion(self.params, lr=self.lr, betas=(self.beta1, self.beta2), weight_decay=self.weight_decay)
        else:
            raise ValueError("unknown optimisation method %r" % self.method)

    # -- schedule ---------------------------------------------------------------------------------
    def current_lr(self) -> float:
        return learning_rate_at(self._step, self.opt, self.init_lr) * self._epoch_decay

    get_learning_rate = current_lr
    getLearningRate = current_lr

    def update_epoch(self, epoch: int):
        if self.update_method == "regular" and self.lr_decay < 1.0 and epoch >= self.start_decay_at:
            self._epoch_decay *= self.lr_decay

    # -- step -------------------------------------------------------------------------------------
    def write_hyper(self, grad_scale: float = 1.0, zero_grad: bool = True):
        """Upload this step's scalars (step count already advanced) into the device struct."""
        t = self._step
        h = self._hyper_host
        h[0], h[1], h[2], h[3] = self.current_lr(), self.beta1, self.beta2, self.eps
        h[4] = self.weight_decay
        h[5] = 1.0 - self.beta1 ** t
        h[6] = 1.0 - self.beta2 ** t
        h[7] = grad_scale
        h[8] = self.max_grad_norm if self.max_grad_norm and self.max_grad_norm > 0 else 0.0
        ints = h.view(torch.int32)
        ints[9] = 1 if self.weight_decay > 0 else 0
        ints[10] = 1 if zero_grad else 0
        self.hyper.copy_(h, non_blocking=True)

    def attach_distributed(self, fused_reducer) -> None:
        """Route the fused update through the peer-memory kernels (sharded master slice and moments)."""
        self.distributed = fused_reducer
        self.exp_avg = self.exp_avg_sq = None      # the replicated moments are not needed any more

    def launch_fused(self):
        """Enqueue norm + update kernels (graph-capturable: reads only device-resident scalars).  With a dynamic loss
        scale (``self.loss_scaler``) the gradient factor is divided by the scale on the device first, and the scale is
        adjusted from the step's non-finite flag afterwards."""
        sc = getattr(self, "loss_scaler", None)
        if sc is not None:
            sc.prepare(self.hyper)
        if getattr(self, "distributed", None) is not None:
            self.distributed.launch()
            if sc is not None:
                sc.update(norm=self.distributed.norm)
            return
        self._launch_local()
        if sc is not None:
            sc.update(nonfinite=self.nonfinite)

    def _launch_local(self):
        s = self.store
        self.grad_sq.zero_()
        self.nonfinite.zero_()
        e = ops.ext()
        n = self.n_update
        if n == s.total:
            e.sq_norm(s.grad, self.grad_sq, self.nonfinite)
            e.adamw_flat(s.master, s.work, s.grad, self.exp_avg, self.exp_avg_sq, self.hyper, self.grad_sq, self.nonfinite)
        elif n > 0:
            e.sq_norm(s.grad[:n], self.grad_sq, self.nonfinite)
            e.adamw_flat(s.master[:n], s.work[:n] if s.work is not None else None, s.grad[:n], self.exp_avg, self.exp_avg_sq,
                         self.hyper, self.grad_sq, self.nonfinite)

    def step(self, grad_scale: float = 1.0, scaler=None):
        """One update.  ``grad_scale`` multiplies the raw gradients (1 / (loss scale * normaliser))."""
        self._step += 1
        if self.fused:
            self.write_hyper(grad_scale)
            self.launch_fused()
            return
        lr = self.current_lr()
        for g in self.optimizer.param_groups:
            g["lr"] = lr
        sc = getattr(self, "loss_scaler", None)
        if sc is not None:
            # torch.optim path (CPU ranks, optimisers without a flat kernel): unscale and test for overflow here
            inv = sc.prepare(None)
            bad = torch.zeros(1, dtype=torch.int32, device=inv.device)
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(inv.to(p.grad.device, p.grad.dtype))
                    if not bool(torch.isfinite(p.grad).all()):
                        bad.fill_(1)
            sc.update(nonfinite=bad)
            if int(bad):
                self._step -= 1          # a skipped step is not counted, as with GradScaler
                return
        if grad_scale != 1.0:
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(grad_scale)
        if self.max_grad_norm and self.max_grad_norm > 0:
            torch.nn.utils.clip_grad_norm_(self.params, self.max_grad_norm)
        if scaler is not None:
            scaler.step(self.optimizer)
        else:
            self.optimizer.step()

    def grad_norm(self) -> float:
        """Global gradient norm of the last fused step (after unscaling), or of ``p.grad`` tensors."""
        if self.fused and getattr(self, "distributed", None) is not None:
            return float(self.distributed.norm.item())
        if self.fused:
            return float(self.grad_sq.sqrt().item()) * float(self._hyper_host[7])
        sq = sum(float(p.grad.float().pow(2).sum()) for p in self.params if p.grad is not None)
        return math.sqrt(sq)

    def zero_grad(self, set_to_none: bool = True):
        if self.fused:
            return   # the update kernel clears the flat gradient buffer
        self.optimizer.zero_grad(set_to_none=set_to_none)
        if self.store is not None:
            self.store.zero_grad()

    # -- state ------------------------------------------------------------------------------------
    def prepare_state_dict(self):
        """Collective part of ``state_dict``: with a sharded step every rank has to call this (the moments of all
        pieces are gathered into the flat layout on rank 0); a no-op otherwise."""
        d = getattr(self, "distributed", None)
        if self.fused and d is not None:
            self._gathered_moments = d.gather_moments()

    def state_dict(self):
        d = getattr(self, "distributed", None)
        if self.fused and d is not None:
            got = getattr(self, "_gathered_moments", None)
            if got is None:
                if d.world > 1:
                    raise RuntimeError("Optim.prepare_state_dict() must be called on every rank before state_dict()")
                got = d.gather_moments()
            self._gathered_moments = None
            # flat-ordered moments: the file does not depend on the world size or on the sharding mode that wrote it
            sd = {"fused": True, "exp_avg": got[0], "exp_avg_sq": got[1]}
        elif self.fused:
            sd = {"fused": True, "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu()}
        else:
            sd = self.optimizer.state_dict()
        sd["_step"] = self._step
        sd["_epoch_decay"] = self._epoch_decay
        return sd

    def load_state_dict(self, sd):
        sd = dict(sd)
        self._step = sd.pop("_step", 0)
        self._epoch_decay = sd.pop("_epoch_decay", 1.0)
        if self.fused and getattr(self, "distributed", None) is not None:
            if "exp_avg" not in sd:
                raise RuntimeError("the checkpoint holds no flat-ordered Adam moments (keys: %s); a sharded run cannot restore "
                                   "its optimiser state from it - resume with -reset_optim" % sorted(sd.keys()))
            self.distributed.load_moments(sd["exp_avg"], sd["exp_avg_sq"])
        elif self.fused:
            if sd.get("fused") and "exp_avg" in sd:
                n = min(self.exp_avg.numel(), sd["exp_avg"].numel())
                self.exp_avg[:n].copy_(sd["exp_avg"][:n])
                self.exp_avg_sq[:n].copy_(sd["exp_avg_sq"][:n])
            elif "state" in sd:
                # a torch.optim state dict (per-parameter moments): scatter into the flat buffers
                for i, p in enumerate(self.params):
                    st = sd["state"].get(i)
                    if st is None:
                        continue
                    off = self.store.offsets[[id(q) for q in self.store.params].index(id(p))]
                    self.exp_avg[off:off + p.numel()].copy_(st["exp_avg"].reshape(-1))
                    self.exp_avg_sq[off:off + p.numel()].copy_(st["exp_avg_sq"].reshape(-1))
        else:
            sd.pop("fused", None)
            if "state" in sd:
                self.optimizer.load_state_dict(sd)
