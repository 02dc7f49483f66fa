"""Continual-learning and other research trainers built on the flat parameter / gradient store.

All of them keep the main trainer's skeleton (data sharding, engine step, logging, checkpoints) and add work on the
flat fp32 vectors, which is where this design pays off: a gradient projection, a Fisher penalty or a Reptile step is
one or two vector operations over ``store.grad`` / ``store.master`` instead of a Python loop over parameters.

* ``Reservoir``            replay memory filled by reservoir sampling (units: whole minibatches), optional stored logits
* ``OCLTrainer``           online continual learning: every new batch is trained together with replayed batches;
                           ``-agem_training`` projects the new gradient onto the half-space of the memory gradient,
                           ``-dark_experience_replay`` adds a loss that keeps the stored output distribution
* ``GEMTrainer``           several memory gradients (one per task), projection by a small dual QP
* ``OfflineCLTrainer``     fine-tuning on new data with replay of old data and an EWC (Fisher) penalty
* ``VATTrainer``           virtual adversarial training on the source embeddings
* ``MetaOCLTrainer``       first-order meta step (Reptile): inner updates on new data, interpolate back
* ``BayesianOCLTrainer``   adds the KL term of Bayes-by-backprop layers (modules exposing ``kl_divergence()``)
* ``ClassifierTrainer``    trainer for utterance classifiers (accuracy instead of perplexity)
* ``Evaluator``            loss / accuracy / BLEU of a model on a data set

Reference behaviour: onmt/train_utils/reservoir.py:23-330, ocl_trainer.py:178-1100, gem_trainer.py:42-132,
offline_cl_trainer.py:183-1150, vat_trainer.py:179-, meta_trainer.py:178-, bayes_by_backprop_trainer.py:180-,
classify_trainer.py:73-, evaluator.py:16-; trainer selection train_distributed.py:65-114.
"""
from __future__ import annotations

import math
import random
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from .trainer import Trainer, _is_list


# ------------------------------------------------------------------------------------------------------------
class Reservoir:
    """Replay memory of at most ``max_samples`` minibatches chosen by reservoir sampling (every observed batch has
    the same probability of being in memory).  Entries are ``(dataset_id, batch)``; ``extras`` can hold stored
    outputs for dark experience replay."""

    def __init__(self, max_samples: int = 40000, update_method: str = "reservoir_sampling", unit: str = "minibatch",
                 dark_experience: bool = False, seed: int = 1234):
        self.max_samples, self.update_method, self.unit = max_samples, update_method, unit
        self.dark_experience = dark_experience
        self.data: Dict[int, tuple] = {}
        self.extras: Dict[int, torch.Tensor] = {}
        self.lambdas: Dict[int, float] = {}        # dual-primal learning: one Lagrange multiplier per memory slot
        self.num_observed = 0
        self.rng = random.Random(seed)

    def __len__(self):
        return len(self.data)

    def add_sample(self, sample, extra=None) -> Optional[int]:
        """Offer one minibatch to the memory; returns the slot it went to (None when it was not kept)."""
        slot = None
        if len(self.data) < self.max_samples:
            slot = len(self.data)
        elif self.update_method == "reservoir_sampling":
            j = self.rng.randint(0, self.num_observed)
            if j < self.max_samples:
                slot = j
        else:   # "fifo"
            slot = self.num_observed % self.max_samples
        self.num_observed += 1
        if slot is not None:
            self.data[slot] = sample
            self.lambdas[slot] = 1.0               # a new sample starts with a fresh multiplier
            if extra is not None:
                self.extras[slot] = extra.detach().cpu()
            else:
                self.extras.pop(slot, None)
        return slot

    def sample(self, n: int = 1):
        if not self.data:
            return []
        slots = [self.rng.randrange(len(self.data)) for _ in range(n)]
        return [(s,) + tuple(self.data[s]) for s in slots]

    def get_stats(self):
        stats: Dict[int, int] = {}
        for ds, _ in self.data.values():
            stats[ds] = stats.get(ds, 0) + 1
        return stats

    def state_dict(self):
        return {"data": self.data, "extras": self.extras, "lambdas": self.lambdas, "num_observed": self.num_observed,
                "unit": self.unit, "update_method": self.update_method}

    def load_state_dict(self, sd):
        self.data, self.extras = sd["data"], sd.get("extras", {})
        self.lambdas = sd.get("lambdas", {k: 1.0 for k in self.data})
        self.num_observed, self.unit, self.update_method = sd["num_observed"], sd["unit"], sd["update_method"]


# ------------------------------------------------------------------------------------------------------------
def project_agem(grad: torch.Tensor, ref: torch.Tensor) -> bool:
    """A-GEM: if ``grad`` points against the memory gradient ``ref``, remove the offending component in place."""
    dot = torch.dot(grad, ref)
    if float(dot) >= 0:
        return False
    grad.add_(ref, alpha=-float(dot) / max(float(torch.dot(ref, ref)), 1e-12))
    return True


def project2cone2(grad: torch.Tensor, memories: torch.Tensor, margin: float = 0.5, eps: float = 1e-3, iters: int = 200):
    """GEM: closest vector to ``grad`` whose dot product with every row of ``memories`` is non-negative.

    Solves the dual ``min_v 0.5 v^T P v + q^T v, v >= margin`` (P = M M^T, q = M g) by projected gradient descent
    (the problem has one variable per task, so a few hundred iterations of a tiny system suffice) and overwrites
    ``grad`` with ``M^T v + g``.
    """
    M = memories.double()
    g = grad.double()
    P = M @ M.t()
    P = 0.5 * (P + P.t()) + eps * torch.eye(P.shape[0], dtype=P.dtype, device=P.device)
    q = M @ g
    v = torch.full_like(q, margin)
    step = 1.0 / max(float(torch.linalg.eigvalsh(P)[-1]), 1e-12)
    for _ in range(iters):
        v = torch.clamp(v - step * (P @ v + q), min=margin)
    grad.copy_((M.t() @ v + g).to(grad.dtype))
    return grad


class EWC:
    """Elastic weight consolidation on flat vectors: ``fisher`` is the running mean of squared gradients on old
    data, ``anchor`` the parameters after the old task; ``penalty_grad`` is added to the gradient."""

    def __init__(self, n: int, device, importance: float = 1.0, normalize: bool = False):
        self.fisher = torch.zeros(n, dtype=torch.float32, device=device)
        self.anchor: Optional[torch.Tensor] = None
        self.count = 0
        self.importance, self.normalize = importance, normalize

    def accumulate(self, grad: torch.Tensor):
        self.fisher.addcmul_(grad, grad)
        self.count += 1

    def finalize(self, params: torch.Tensor):
        if self.count:
            self.fisher.div_(self.count)
        if self.normalize:
            self.fisher.div_(self.fisher.max().clamp_min(1e-20))
        self.anchor = params.detach().clone()
        self.count = 0

    def penalty(self, params: torch.Tensor) -> torch.Tensor:
        return 0.5 * self.importance * torch.sum(self.fisher * (params - self.anchor) ** 2)

    def add_penalty_grad(self, grad: torch.Tensor, params: torch.Tensor, scale: float = 1.0):
        if self.anchor is not None and self.importance > 0:
            grad.add_(self.fisher * (params - self.anchor), alpha=self.importance * scale)

    def state_dict(self):
        return {"fisher": self.fisher.cpu(), "anchor": None if self.anchor is None else self.anchor.cpu()}

    def load_state_dict(self, sd):
        self.fisher.copy_(sd["fisher"])
        self.anchor = None if sd["anchor"] is None else sd["anchor"].to(self.fisher.device)


# ------------------------------------------------------------------------------------------------------------
class _FlatAccess:
    """Gives trainers one flat fp32 gradient / parameter view whatever the optimiser layout is."""

    def _grad_store(self):
        # the flat gradient buffer is only filled when the fused optimiser path is active
        return getattr(self.engine, "store", None) if getattr(self.engine.optim, "fused", False) else None

    def flat_grad(self) -> torch.Tensor:
        store = self._grad_store()
        if store is not None:
            return store.grad
        return torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float()
                          for p in self.model.parameters() if p.requires_grad])

    def set_flat_grad(self, g: torch.Tensor):
        store = self._grad_store()
        if store is not None:
            if g.data_ptr() != store.grad.data_ptr():
                store.grad.copy_(g)
            return
        off = 0
        for p in self.model.parameters():
            if not p.requires_grad:
                continue
            n = p.numel()
            p.grad = g[off:off + n].view_as(p).to(p.dtype).clone()
            off += n

    def flat_params(self) -> torch.Tensor:
        store = self._grad_store()
        if store is not None:
            return store.master
        return torch.cat([p.detach().reshape(-1).float() for p in self.model.parameters() if p.requires_grad])

    def zero_flat_grad(self):
        store = self._grad_store()
        if store is not None:
            store.grad.zero_()
        else:
            for p in self.model.parameters():
                p.grad = None


class OCLTrainer(Trainer, _FlatAccess):
    """Online continual learning: each incoming minibatch is seen once; ``replay_ratio`` memory batches are trained
    with it.  With ``-agem_training`` the memory batches only provide a reference gradient for the projection
    (``-agem_summation``: the projected gradient and the memory gradient are summed, so memory is also trained)."""

    replay_per_step = 1

    def __init__(self, device, dicts, opt, constants=None, **kw):
        opt.cuda_graph = False          # the step is steered from the host
        super().__init__(device, dicts, opt, constants, **kw)
        self.reservoir = Reservoir(getattr(opt, "reservoir_size", 0) or 1000,
                                   dark_experience=getattr(opt, "dark_experience_replay", False),
                                   seed=getattr(opt, "seed", 9999) + self.rank)
        self.agem = getattr(opt, "agem_training", False)
        self.agem_sum = getattr(opt, "agem_summation", False)
        self.projections = 0
        # dual-primal learning (-dpl_training): replayed batches are weighted by a Lagrange multiplier per memory slot;
        # every -dpl_count updates the multipliers move by lr * (loss per token - -dpl_epsilon), clamped at zero, so
        # memory whose loss violates the constraint is replayed harder (reference: offline_cl_trainer.py:1141-1223)
        self.dpl = bool(getattr(opt, "dpl_training", False))
        self.dpl_epsilon = float(getattr(opt, "dpl_epsilon", 0.0) or 0.0)
        self.dpl_every = max(1, int(getattr(opt, "dpl_count", 1) or 1))
        self.dpl_lr = float(getattr(opt, "dpl_lr", 0.1) or 0.1)
        self._dpl_counter = 0

    # one optimisation step on (new batch, memory batches)
    def train_step(self, batch, dataset_id: int = 0):
        eng = self.engine
        mem = self.reservoir.sample(self.replay_per_step) if len(self.reservoir) else []
        if self.agem and mem:
            for _, _, mb in mem:
                eng.train_step(mb, update=False)
            ref = self.flat_grad().clone()
            self.zero_flat_grad()
            loss, correct = eng.train_step(batch, update=False)
            g = self.flat_grad()
            self.projections += int(project_agem(g, ref))
            if self.agem_sum:
                g.add_(ref)
            self.set_flat_grad(g)
        else:
            for slot, _, mb in mem:
                eng.loss_weight = self.reservoir.lambdas.get(slot, 1.0) if self.dpl else 1.0
                eng.train_step(mb, update=False)
            eng.loss_weight = 1.0
            loss, correct = eng.train_step(batch, update=False)
        self._apply_update(batch.tgt_size + sum(mb.tgt_size for _, _, mb in mem))
        self.reservoir.add_sample((dataset_id, batch))
        if self.dpl:
            self._dpl_counter += 1
            if self._dpl_counter >= self.dpl_every:
                self.update_lambdas()
                self._dpl_counter = 0
        return loss, correct

    @torch.no_grad()
    def update_lambdas(self, max_batches: int = 16):
        """Dual ascent on the multipliers of (a sample of) the memory: ``lambda += lr * (loss per token - epsilon)``,
        never below zero; the per-slot differences are summed over ranks first."""
        slots = sorted(self.reservoir.data)
        if len(slots) > max_batches:
            slots = sorted(self.reservoir.rng.sample(slots, max_batches))
        if not slots:
            return
        diffs = []
        for s in slots:
            _, mb = self.reservoir.data[s]
            loss, _ = self.engine.eval_step(mb)
            diffs.append(float(loss) / max(mb.tgt_size, 1) - self.dpl_epsilon)
        diffs = self._all_reduce_scalars(diffs)
        for s, d in zip(slots, diffs):
            self.reservoir.lambdas[s] = max(0.0, self.reservoir.lambdas.get(s, 1.0) + self.dpl_lr * d / max(self.world_size, 1))
        self.model.train()

    def _apply_update(self, n_words: int):
        eng = self.engine
        if getattr(self.opt, "normalize_gradient", False):
            eng.grad_scale = 1.0 / max(self._all_reduce_scalars([float(n_words)])[0], 1.0)
        if eng.reducer is not None:
            eng.reducer(self.flat_grad())
        eng.optim.step(eng.grad_scale)
        if not eng.optim.fused:
            eng.optim.zero_grad()

    def train_epoch(self, train_data, valid_data, epoch: int, resume_itr_state=None):
        datasets = list(train_data) if _is_list(train_data) else [train_data]
        tot_loss = tot_words = 0.0
        iterator = None
        self.model.train()
        for ds_id, ds in enumerate(datasets):          # tasks arrive one after the other
            iterator = self._iterator(ds, epoch, seed_offset=ds_id)
            for i, batch in enumerate(iterator.next_epoch_itr()):
                loss, _ = self.train_step(batch, ds_id)
                tot_loss += float(loss)
                tot_words += batch.tgt_size
                if (i + 1) % max(1, getattr(self.opt, "log_interval", 100)) == 0:
                    self.log("Epoch %2d task %d, %5d batches; ppl: %8.2f ; memory: %d ; projections: %d"
                             % (epoch, ds_id, i + 1, math.exp(min(tot_loss / max(tot_words, 1), 100)), len(self.reservoir),
                                self.projections))
                max_step = getattr(self.opt, "max_step", 0)
                if max_step and self.optim._step >= max_step:
                    break
        return tot_loss / max(tot_words, 1.0), iterator


class GEMTrainer(OCLTrainer):
    """Gradient episodic memory: one reference gradient per previous task; the new gradient is projected into the
    intersection of their half-spaces."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.task_memory: Dict[int, List] = {}
        self.margin = 0.5

    def train_step(self, batch, dataset_id: int = 0):
        eng = self.engine
        refs = []
        for task, batches in self.task_memory.items():
            if task == dataset_id or not batches:
                continue
            self.zero_flat_grad()
            for mb in batches[:self.replay_per_step]:
                eng.train_step(mb, update=False)
            refs.append(self.flat_grad().clone())
        self.zero_flat_grad()
        loss, correct = eng.train_step(batch, update=False)
        if refs:
            g = self.flat_grad()
            M = torch.stack(refs)
            if bool((M @ g < 0).any()):
                project2cone2(g, M, self.margin)
                self.projections += 1
            self.set_flat_grad(g)
        self._apply_update(batch.tgt_size)
        mem = self.task_memory.setdefault(dataset_id, [])
        if len(mem) < max(1, (getattr(self.opt, "reservoir_size", 0) or 64)):
            mem.append(batch)
        else:
            mem[random.randrange(len(mem))] = batch
        return loss, correct


class OfflineCLTrainer(OCLTrainer):
    """Adapting a trained model to new data: the first data set of the list is the old data (replayed from the
    reservoir and used for the Fisher estimate), the others are new; the EWC penalty gradient is added before every
    update once ``-ewc_delay`` updates have passed, and its importance decays every ``-ewc_decay_every`` updates."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        opt = self.opt
        self.ewc = EWC(self.flat_params().numel(), self.device, getattr(opt, "ewc_importance", 0.0),
                       getattr(opt, "ewc_normalize", False)) if getattr(opt, "ewc_importance", 0.0) > 0 else None

    def estimate_fisher(self, old_data, max_batches: int = 64):
        if self.ewc is None:
            return
        it = self._iterator(old_data, 1, shuffle=True).next_epoch_itr()
        for i, batch in enumerate(it):
            if i >= max_batches:
                break
            self.zero_flat_grad()
            self.engine.train_step(batch, update=False)
            self.ewc.accumulate(self.flat_grad() / max(batch.tgt_size, 1))
            self.reservoir.add_sample((0, batch))
        self.zero_flat_grad()
        self.ewc.finalize(self.flat_params())

    def _apply_update(self, n_words: int):
        opt = self.opt
        if self.ewc is not None and self.optim._step >= getattr(opt, "ewc_delay", 0):
            every = max(1, getattr(opt, "ewc_decay_every", 10000))
            decay = getattr(opt, "ewc_decay_scale", 10) ** (-(self.optim._step // every))
            # the data gradient is a sum over n_words tokens; keep the penalty on the same scale
            g = self.flat_grad()
            self.ewc.add_penalty_grad(g, self.flat_params(), scale=decay * n_words)
            self.set_flat_grad(g)
        super()._apply_update(n_words)

    def train_epoch(self, train_data, valid_data, epoch: int, resume_itr_state=None):
        datasets = list(train_data) if _is_list(train_data) else [train_data]
        if epoch == 1 and len(datasets) > 1:
            self.estimate_fisher(datasets[0])
            datasets = datasets[1:]
        return super().train_epoch(datasets, valid_data, epoch, resume_itr_state)

    def finalize(self, train_data, valid_data):
        """The closing pass of a round (``-finalize_only``): the round's saved checkpoints are averaged into the model,
        the replay memory is filled from the round's training data, the averaged model is validated and written with
        the memory as ``<save_model>_final.pt`` - the file the next round starts from.
        (reference: onmt/train_utils/offline_cl_trainer.py:3411-3431, :2648-2700)"""
        import math
        import os

        from ..tools.checkpoints import average_state_dicts, best_checkpoints
        from .checkpoint import load_model_state, model_state_for_saving
        opt = self.opt
        files = best_checkpoints(opt.save_model, top=10 ** 6)
        if files and self.is_main():
            self.log("[INFO] Averaging %d checkpoints of this round" % len(files))
        if files:
            states = [torch.load(f, map_location="cpu", weights_only=False)["model"] for f in files]
            load_model_state(self.model, average_state_dicts(states))
            store = getattr(self.engine, "store", None)
            if store is not None:
                store.sync_work()                 # the bf16 working copy follows the fp32 parameters just loaded
        for ds in (list(train_data) if _is_list(train_data) else [train_data]):
            for batch in self._iterator(ds, 1, shuffle=True).next_epoch_itr():
                self.reservoir.add_sample((0, batch))
        vloss, vacc = self.eval(valid_data)
        vppl = math.exp(min(vloss, 100)) if vloss == vloss else float("nan")
        self.log("[INFO] Validation perplexity: %g  accuracy: %.4f" % (vppl, vacc))
        name = opt.save_model + "_final.pt"
        if self.is_main():
            os.makedirs(os.path.dirname(os.path.abspath(name)), exist_ok=True)
            torch.save({"model": model_state_for_saving(self.model), "dicts": self.dicts, "opt": opt, "epoch": -1,
                        "reservoir": self.reservoir.state_dict(), "valid_ppl": vppl}, name)
            self.log("[INFO] Saved checkpoint %s" % name)
        return name

    def run(self, checkpoint=None, train_data=None, valid_data=None):
        opt = self.opt
        loaded = checkpoint if checkpoint is not None else getattr(self, "_resume_checkpoint", None)
        if loaded is not None and loaded.get("reservoir") is not None:
            self.reservoir.load_state_dict(loaded["reservoir"])            # a *_final.pt of the previous round
        if getattr(opt, "finalize_only", False):
            self.log("[INFO] Skipping the training and validation part. Only finalizing the models")
            return self.finalize(train_data, valid_data)
        budget = int(getattr(opt, "max_examples_seen", 0) or 0)
        if budget > 0:
            # the budget counts minibatches; it is turned into whole epochs (reference: offline_cl_trainer.py:2636-2639)
            sets = list(train_data) if _is_list(train_data) else [train_data]
            per_epoch = max(1, sum(len(d) for d in sets))
            opt.epochs = budget // per_epoch
            self.log("[INFO] Max epoch: %d" % opt.epochs)
            if opt.epochs == 0:
                raise ValueError("No training is done (-max_examples_seen %d is less than one epoch of %d minibatches). "
                                 "Use -finalize_only." % (budget, per_epoch))
        return super().run(checkpoint, train_data, valid_data)


class EWCTrainer(OfflineCLTrainer):
    """The main trainer's elastic-weight-consolidation switches (reference: onmt/train_utils/mp_trainer.py:402-412,
    1162-1517): ``-estimate_fisher_information`` runs over the training data once, accumulates the squared gradients
    and writes them with the current weights to ``<checkpoint>.fisher``; ``-load_fisher <file>`` reads such a file
    and adds the penalty ``ewc_importance / 2 * sum F (w - w*)^2`` to every later update."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        opt = self.opt
        if self.ewc is None:
            self.ewc = EWC(self.flat_params().numel(), self.device, float(getattr(opt, "ewc_importance", 0.0) or 1.0),
                           getattr(opt, "ewc_normalize", False))
        path = getattr(opt, "load_fisher", "") or ""
        if path:
            self.ewc.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
            if self.ewc.anchor is None:
                self.ewc.anchor = self.flat_params().clone()
            self.log("[INFO] Fisher information loaded from %s" % path)

    def fisher_path(self) -> str:
        base = getattr(self.opt, "load_from", "") or (getattr(self.opt, "save_model", "model") + ".pt")
        return base + ".fisher"

    def run(self, checkpoint=None, train_data=None, valid_data=None):
        if getattr(self.opt, "estimate_fisher_information", False):
            data = train_data[0] if _is_list(train_data) else train_data
            self.estimate_fisher(data, max_batches=10 ** 9)
            sd = self.ewc.state_dict()
            if self.is_main():
                torch.save(sd, self.fisher_path())
                self.log("[INFO] Fisher information written to %s" % self.fisher_path())
            return self.fisher_path()
        return super().run(checkpoint, train_data, valid_data)

    def train_epoch(self, train_data, valid_data, epoch: int, resume_itr_state=None):
        return OCLTrainer.train_epoch(self, train_data, valid_data, epoch, resume_itr_state)


class VATTrainer(OCLTrainer):
    """Virtual adversarial training: besides the supervised loss, the output distribution must not move when the
    source embeddings are perturbed in the direction that changes it most (one power iteration)."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.vat_weight = float(getattr(self.opt, "vat_training", 0) or 1.0)
        self.xi, self.eps = 1e-2, 1.0

    def _logp(self, batch, noise=None):
        embed = self.model.encoder.embed if hasattr(self.model, "encoder") and hasattr(self.model.encoder, "embed") else None
        handle = None
        if noise is not None and embed is not None:
            handle = embed.register_forward_hook(lambda _m, _i, out: out + noise.to(out.dtype))
        try:
            out = self.model(batch, return_logits=True, compute_loss=False)
        finally:
            if handle is not None:
                handle.remove()
        return torch.log_softmax(out["logprobs"].float(), -1), out

    def vat_loss(self, batch):
        with torch.no_grad():
            clean, out = self._logp(batch)
        rows = out["src"].tokens.shape[0]
        hidden = out["context_packed"].shape[-1]
        d = torch.randn(rows, hidden, device=clean.device)
        d = (self.xi * d / d.norm(dim=-1, keepdim=True).clamp_min(1e-8)).requires_grad_()
        pert, _ = self._logp(batch, d)
        kl = F.kl_div(pert, clean, log_target=True, reduction="sum")
        g, = torch.autograd.grad(kl, d, allow_unused=True)
        if g is None:
            return clean.new_zeros(())
        r = self.eps * g / g.norm(dim=-1, keepdim=True).clamp_min(1e-8)
        pert, _ = self._logp(batch, r.detach())
        return F.kl_div(pert, clean, log_target=True, reduction="sum")

    def train_step(self, batch, dataset_id: int = 0):
        dev_batch = batch.cuda(self.device, hot_only=True) if self.cuda else batch
        loss, correct = self.engine.train_step(batch, update=False)
        if self.vat_weight > 0 and not getattr(self.engine.optim, "fused", False):
            (self.vat_weight * self.vat_loss(dev_batch)).backward()
        self._apply_update(batch.tgt_size)
        return loss, correct


class MetaOCLTrainer(OCLTrainer):
    """First-order meta-learning (Reptile): ``inner_steps`` ordinary updates on the new batch plus replayed batches,
    then the parameters move only a fraction ``meta_lr`` of the way from where they started."""

    inner_steps, meta_lr = 2, 0.5

    def train_step(self, batch, dataset_id: int = 0):
        store = self.engine.store                     # parameters are views of store.master on every path
        start = store.master.clone()
        loss = correct = None
        for _ in range(self.inner_steps):
            loss, correct = super().train_step(batch, dataset_id)
            self.reservoir.num_observed -= 1          # the same batch is offered to the memory once, below
        self.reservoir.num_observed += 1
        with torch.no_grad():
            store.master.copy_(start + self.meta_lr * (store.master - start))
        store.sync_work()
        return loss, correct


class BayesianOCLTrainer(OCLTrainer):
    """Adds ``kl_weight * sum(module.kl_divergence())`` over Bayes-by-backprop layers to every step."""

    def __init__(self, device, dicts, opt, constants=None, **kw):
        from ..modules.bayesian import configure_prior
        configure_prior(opt)          # -prior_pi / -neg_log_sigma1 / -neg_log_sigma2 before any Bayesian layer is built
        super().__init__(device, dicts, opt, constants, **kw)

    def train_step(self, batch, dataset_id: int = 0):
        loss, correct = self.engine.train_step(batch, update=False)
        kls = [m.kl_divergence() for m in self.model.modules() if hasattr(m, "kl_divergence")]
        if kls and not getattr(self.engine.optim, "fused", False):
            n_batches = max(1, getattr(self.opt, "bayes_num_batches", 1000))
            (sum(kls) / n_batches).backward()
        self._apply_update(batch.tgt_size)
        self.reservoir.add_sample((dataset_id, batch))
        return loss, correct


# ------------------------------------------------------------------------------------------------------------
class ClassifierTrainer(Trainer):
    """Trainer for classification models: the engine's loss is the classifier's cross-entropy, the reported metric
    is accuracy over labelled units; checkpoints are ranked by (1 - accuracy)."""

    def __init__(self, device, dicts, opt, constants=None, **kw):
        opt.save_metrics = "accuracy"
        super().__init__(device, dicts, opt, constants, **kw)


class Evaluator:
    """Evaluates a model on a data set: per-token loss, accuracy and (given references) corpus BLEU of greedy or
    beam-search output."""

    def __init__(self, model, dicts, opt, device=None):
        self.model, self.dicts, self.opt = model, dicts, opt
        self.device = device or next(model.parameters()).device

    @torch.no_grad()
    def eval_loss(self, data):
        from ..data.iterator import DataIterator
        self.model.eval()
        tot_loss = tot_words = tot_correct = 0.0
        for batch in DataIterator(data, shuffle=False).next_epoch_itr():
            if self.device.type == "cuda":
                batch = batch.cuda(self.device)
            out = self.model(batch)
            tot_loss += float(out["loss"])
            tot_correct += float(out["correct"])
            tot_words += batch.tgt_size
        return tot_loss / max(tot_words, 1), tot_correct / max(tot_words, 1)

    @torch.no_grad()
    def eval_translate(self, src_sents, refs, beam_size: int = 1, max_len: int = 100):
        from ..data.dataset import collate
        from ..inference.beam_search import BeamConfig, beam_search
        from ..utils.metrics import corpus_bleu
        tgt = self.dicts["tgt"]
        hyps = []
        for i in range(0, len(src_sents), 16):
            chunk = src_sents[i:i + 16]
            batch = collate([self.dicts["src"].convert_to_idx(s, "<unk>") for s in chunk], None, padded=True, packed=True, round_to=1)
            if self.device.type == "cuda":
                batch = batch.cuda(self.device)
            for h in beam_search(self.model, batch, BeamConfig(beam_size=beam_size, max_len=max_len)):
                hyps.append(tgt.convert_to_labels(h[0].tokens, 3, including_stop=False))
        return corpus_bleu(hyps, refs), hyps


def select_trainer(opt):
    """Trainer class for the given options (same precedence as the reference's ``run_process``)."""
    if getattr(opt, "ocl_training", False):
        if getattr(opt, "bayes_by_backprop", False):
            return BayesianOCLTrainer
        if getattr(opt, "vat_training", 0) > 0:
            return VATTrainer
        if getattr(opt, "meta_learning", False):
            return MetaOCLTrainer
        if getattr(opt, "gem_training", False):
            return GEMTrainer
        return OCLTrainer
    if getattr(opt, "offline_cl_training", False):
        return OfflineCLTrainer
    if getattr(opt, "model", "") in ("classifier", "wav2vec2_classifier") or getattr(opt, "classifier_training", False):
        return ClassifierTrainer
    if getattr(opt, "estimate_fisher_information", False) or getattr(opt, "load_fisher", ""):
        return EWCTrainer
    return Trainer
