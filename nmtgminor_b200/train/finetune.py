"""Fine-tuning utilities used for the Whisper / pretrained-model recipes: LoRA adapters on the fused Linear layers,
an exponential moving average of the parameters kept on the flat fp32 vector, teacher-student distillation, and a
batch-ensemble wrapper.

Reference: whisper/whisper_lora.py / the memory-efficient and EMA trainers of whisper/*.py (Hugging Face
``Seq2SeqTrainer`` subclasses; here the same pieces plug into this framework's ``Trainer``), distillation loss
onmt/modules/loss.py (KL term), batch ensemble onmt/modules/batch_ensemble/.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..models.layers import Linear


class LoRALinear(nn.Module):
    """``y = base(x) + (alpha / r) * (dropout(x) A^T) B^T`` with the base weight frozen.

    The two low-rank products run through the same fused GEMM as the base layer (rank is rounded up to a multiple of
    8 so that every leading dimension stays 16-byte aligned)."""

    def __init__(self, base: Linear, r: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base = base
        r = (r + 7) // 8 * 8
        out_dim, in_dim = base.weight.shape
        self.lora_a = Linear(in_dim, r, bias=False)
        self.lora_b = Linear(r, out_dim, bias=False)
        nn.init.kaiming_uniform_(self.lora_a.weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_b.weight)
        self.scaling = alpha / r
        self.dropout = dropout
        for p in base.parameters():
            p.requires_grad_(False)

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def forward(self, x, *args, **kw):
        y = self.base(x, *args, **kw)
        xd = F.dropout(x, self.dropout, self.training) if self.dropout > 0 else x
        return y + self.scaling * self.lora_b(self.lora_a(xd)).to(y.dtype)

    @torch.no_grad()
    def merged_weight(self):
        return self.base.weight + self.scaling * (self.lora_b.weight @ self.lora_a.weight)


def apply_lora(model: nn.Module, r: int = 8, alpha: float = 16.0, dropout: float = 0.0, target: Iterable[str] = ("q", "kv", "qkv", "out"),
               freeze_rest: bool = True) -> List[str]:
    """Replace the named ``Linear`` children (by attribute name) with ``LoRALinear``; returns the replaced paths."""
    target = set(target)
    replaced = []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            if child_name in target and isinstance(child, Linear):
                setattr(module, child_name, LoRALinear(child, r, alpha, dropout))
                replaced.append((name + "." if name else "") + child_name)
    if freeze_rest:
        for n, p in model.named_parameters():
            p.requires_grad_("lora_" in n)
    return replaced


@torch.no_grad()
def merge_lora(model: nn.Module) -> int:
    """Fold every adapter into its base weight and restore plain ``Linear`` modules; returns how many were merged."""
    n = 0
    for module in list(model.modules()):
        for child_name, child in list(module.named_children()):
            if isinstance(child, LoRALinear):
                child.base.weight.copy_(child.merged_weight())
                setattr(module, child_name, child.base)
                n += 1
    return n


class FlatEMA:
    """Exponential moving average of all parameters as ONE vector operation on the flat fp32 master buffer
    (``store.master``), or on a list of parameters when no flat store is given."""

    def __init__(self, params_or_store, decay: float = 0.999):
        self.decay = decay
        self.store = params_or_store if hasattr(params_or_store, "master") else None
        if self.store is not None:
            self.shadow = self.store.master.detach().clone()
        else:
            self.params = [p for p in params_or_store]
            self.shadow = [p.detach().clone() for p in self.params]
        self.backup = None

    @torch.no_grad()
    def update(self, step: Optional[int] = None):
        d = self.decay if step is None else min(self.decay, (1 + step) / (10 + step))
        if self.store is not None:
            self.shadow.lerp_(self.store.master, 1 - d)
        else:
            for s, p in zip(self.shadow, self.params):
                s.lerp_(p.detach(), 1 - d)

    @torch.no_grad()
    def swap_in(self):
        """Evaluate with the averaged weights; ``swap_out`` restores the training weights."""
        if self.store is not None:
            self.backup = self.store.master.clone()
            self.store.master.copy_(self.shadow)
            self.store.sync_work()
        else:
            self.backup = [p.detach().clone() for p in self.params]
            for s, p in zip(self.shadow, self.params):
                p.copy_(s)

    @torch.no_grad()
    def swap_out(self):
        if self.backup is None:
            return
        if self.store is not None:
            self.store.master.copy_(self.backup)
            self.store.sync_work()
        else:
            for b, p in zip(self.backup, self.params):
                p.copy_(b)
        self.backup = None

    def state_dict(self):
        return {"decay": self.decay, "shadow": self.shadow}


def distillation_loss(student_logits, teacher_logits, labels, pad_idx: int = 0, alpha: float = 0.5, temperature: float = 2.0,
                      label_smoothing: float = 0.0):
    """``alpha * T^2 * KL(teacher || student) + (1 - alpha) * CE`` summed over non-pad rows of ``[N, V]`` logits."""
    keep = labels != pad_idx
    s, t = student_logits.float()[keep], teacher_logits.float()[keep].detach()
    kl = F.kl_div(F.log_softmax(s / temperature, -1), F.log_softmax(t / temperature, -1), log_target=True, reduction="sum")
    ce = F.cross_entropy(s, labels[keep], reduction="sum", label_smoothing=label_smoothing)
    return alpha * temperature ** 2 * kl + (1 - alpha) * ce


def distill_step(student, teacher, batch, alpha: float = 0.5, temperature: float = 2.0):
    """One forward pass of both models on ``batch``; returns the combined loss (call ``backward`` on it)."""
    with torch.no_grad():
        t_out = teacher(batch, return_logits=True, compute_loss=False)
    s_out = student(batch, return_logits=True, compute_loss=False)
    tgt = s_out["tgt"]
    unpad = lambda o: ops.reference.unpad_packed(o["logprobs"].transpose(0, 1), tgt.cu, tgt.tokens.shape[0])
    return distillation_loss(unpad(s_out), unpad(t_out), s_out["target"], getattr(student, "pad_idx", 0), alpha, temperature)


class BatchEnsembleLinear(nn.Module):
    """Rank-1 batch ensemble: member m computes ``((x * r_m) W^T) * s_m + b_m`` with one shared weight matrix."""

    def __init__(self, in_dim: int, out_dim: int, members: int = 4, bias: bool = True):
        super().__init__()
        self.shared = Linear(in_dim, out_dim, bias=False)
        self.r = nn.Parameter(torch.ones(members, in_dim) + 0.1 * torch.randn(members, in_dim))
        self.s = nn.Parameter(torch.ones(members, out_dim) + 0.1 * torch.randn(members, out_dim))
        self.bias = nn.Parameter(torch.zeros(members, out_dim)) if bias else None
        self.members = members

    def forward(self, x, member: Optional[torch.Tensor] = None):
        """x [N, in]; ``member`` [N] picks the ensemble member of every row (default: rows split evenly, in order)."""
        if member is None:
            member = torch.arange(x.shape[0], device=x.device) * self.members // max(x.shape[0], 1)
        y = self.shared((x * self.r[member].to(x.dtype))) * self.s[member].to(x.dtype)
        return y if self.bias is None else y + self.bias[member].to(y.dtype)


class DistillationWrapper(nn.Module):
    """Presents ``student`` to the training engine with the distillation objective as its loss: the engine calls
    ``wrapper(batch, grad_scale=...)`` and back-propagates ``out["loss"]``.  The teacher is held outside the module
    tree, so it is neither trained nor saved."""

    def __init__(self, student: nn.Module, teacher: nn.Module, alpha: float = 0.5, temperature: float = 2.0):
        super().__init__()
        self.student = student
        self._teacher = [teacher.eval()]
        self.alpha, self.temperature = alpha, temperature
        for p in teacher.parameters():
            p.requires_grad_(False)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("student"), name)

    def forward(self, batch, grad_scale=None, **kw):
        if not self.training:
            return self.student(batch, **kw)
        with torch.no_grad():
            t_out = self._teacher[0](batch, return_logits=True, compute_loss=False)
        s_out = self.student(batch, return_logits=True, compute_loss=False)
        tgt = s_out["tgt"]
        unpad = lambda o: ops.reference.unpad_packed(o["logprobs"].transpose(0, 1), tgt.cu, tgt.tokens.shape[0])
        s_logits, labels = unpad(s_out), s_out["target"]
        loss = distillation_loss(s_logits, unpad(t_out), labels, getattr(self.student, "pad_idx", 0), self.alpha, self.temperature)
        keep = labels != getattr(self.student, "pad_idx", 0)
        correct = (s_logits.argmax(-1)[keep] == labels[keep]).sum().float().reshape(1)
        s_out.update(loss=loss.reshape(1), correct=correct)
        return s_out
