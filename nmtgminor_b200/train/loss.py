"""Loss modules with the reference's call signatures.

``NMTLossFunc(outputs, targets)`` returns ``{'loss', 'data', 'correct', 'total', ...}`` like the reference's class
(onmt/modules/loss.py:162-408).  When the model already computed the fused loss (``outputs['loss']``, the normal
training path) it is passed through; otherwise the label-smoothed cross-entropy is evaluated from
``outputs['logprobs']`` (logits ``[T, B, V]``) over ALL non-pad target positions (the reference's B×T / T×B mask
mix-up is not reproduced).  Also here: CTC (``CTCLossFunc``, onmt/modules/loss.py:530, onmt/speech/ctc_loss.py:9-116),
the combined NMT + CTC loss (:611), masked predictive coding (``MPCLoss`` :411), classification
(``ClassifierLoss`` :448), language-model fusion (``FusionLoss`` :660), language-id cross-entropy (onmt/models/speech_recognizer/lid_loss.py:13) and the
KL distillation term used by the continual-learning trainers.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class CrossEntropyLossBase(nn.Module):
    def __init__(self, output_size: int, label_smoothing: float = 0.0, padding_idx: int = 0):
        super().__init__()
        self.output_size, self.label_smoothing, self.padding_idx = output_size, label_smoothing, padding_idx

    def _compute_loss(self, logits, targets):
        """logits [N, V], targets [N] -> (loss_sum, loss_data, n_correct)."""
        smoothing = self.label_smoothing if self.training else 0.0
        loss, correct, _ = ops.cross_entropy(logits, targets, smoothing, self.padding_idx)
        return loss.sum(), float(loss.detach().sum()), correct


class NMTLossFunc(CrossEntropyLossBase):
    def __init__(self, hidden_size: int, output_size: int, label_smoothing: float = 0.0, mirror: bool = False,
                 padding_idx: int = 0, **_unused):
        super().__init__(output_size, label_smoothing, padding_idx)
        self.hidden_size, self.mirror = hidden_size, mirror

    def forward(self, model_outputs, targets, model=None, **_unused):
        if model_outputs.get("loss") is not None:
            loss = model_outputs["loss"].sum()
            total = int((targets != self.padding_idx).sum()) if targets is not None else 0
            # terms of the mirror / reconstruction decoders are already inside the model's loss; they are reported apart
            return {"loss": loss, "data": loss.detach(), "correct": model_outputs.get("correct"), "total": total,
                    "rev_loss": model_outputs.get("rev_loss"), "mirror_loss": model_outputs.get("mirror_loss"),
                    "rec_loss": model_outputs.get("rec_loss")}
        logits = model_outputs["logprobs"]
        flat_logits = logits.reshape(-1, logits.shape[-1])
        flat_targets = targets.reshape(-1)
        if logits.is_cuda and logits.dtype == torch.bfloat16:
            flat_logits = flat_logits.clone()      # the fused kernel overwrites its input with the gradient
        loss, data, correct = self._compute_loss(flat_logits, flat_targets)
        out = {"loss": loss, "data": data, "correct": correct, "total": int((flat_targets != self.padding_idx).sum())}
        if self.mirror and "rev_logprobs" in model_outputs:
            rl = model_outputs["rev_logprobs"]
            rev, rev_data, _ = self._compute_loss(rl.reshape(-1, rl.shape[-1]), model_outputs["rev_target"].reshape(-1))
            hid, rev_hid = model_outputs["hidden"], model_outputs["rev_hidden"]
            mask = (targets != self.padding_idx).unsqueeze(-1)
            mirror = ((hid - rev_hid.flip(0)) * mask).float().pow(2).sum()
            out.update(rev_loss=rev, rev_loss_data=rev_data, mirror_loss=mirror)
        return out


class FusionLoss(CrossEntropyLossBase):
    """Loss of a translation model fused with a frozen language model ("simple fusion", pre-norm variant):
    ``log p = log_softmax(tm_logits + log p_lm)``.  ``model_outputs['tm']['hidden']`` / ``['lm']['hidden']`` are the two
    decoders' states ``[T, B, H]``, ``model`` gives the two output layers (``model.tm_model.generator``,
    ``model.lm_model.generator``); a ``model_outputs['logprobs']`` that already holds the fused log-probabilities is used
    as it is.  Reference: onmt/modules/loss.py:660-737."""

    def forward(self, model_outputs, targets, model=None, backward: bool = False, normalizer: float = 1.0, **_unused):
        flat_targets = targets.reshape(-1)
        keep = (flat_targets != self.padding_idx).nonzero(as_tuple=False).squeeze(1)
        if "tm" in model_outputs and model is not None:
            tm = model_outputs["tm"]["hidden"]
            lm = model_outputs["lm"]["hidden"]
            tm = tm.reshape(-1, tm.shape[-1]).index_select(0, keep)
            lm = lm.reshape(-1, lm.shape[-1]).index_select(0, keep)
            tm_logits = model.tm_model.generator(tm).float()
            with torch.no_grad():
                log_lm = torch.log_softmax(model.lm_model.generator(lm).float(), -1)
            dists = torch.log_softmax(tm_logits + log_lm, -1)
        else:
            lp = model_outputs["logprobs"]
            dists = lp.reshape(-1, lp.shape[-1]).float().index_select(0, keep)
        gold = flat_targets.index_select(0, keep)
        smoothing = self.label_smoothing if self.training else 0.0
        nll = -dists.gather(1, gold[:, None]).squeeze(1)
        loss = ((1.0 - smoothing) * nll - smoothing * dists.mean(-1)).sum() if smoothing > 0 else nll.sum()
        if backward:
            (loss / normalizer).backward()
        return {"loss": loss, "data": float(loss.detach()), "correct": int((dists.argmax(-1) == gold).sum()), "total": int(gold.numel())}


class CTCLossFunc(nn.Module):
    """CTC over encoder states: ``forward(logits [T, B, V], src_lengths, targets [B, U], tgt_lengths)``."""

    def __init__(self, output_size: int = 0, label_smoothing: float = 0.0, blank_idx: int = 0, padding_idx: int = 0,
                 zero_infinity: bool = True):
        super().__init__()
        self.blank, self.pad, self.zero_infinity = blank_idx, padding_idx, zero_infinity
        self.label_smoothing = label_smoothing

    def forward(self, logits, input_lengths, targets, target_lengths=None):
        lp = F.log_softmax(logits.float(), dim=-1)
        if target_lengths is None:
            target_lengths = (targets != self.pad).sum(-1)
        loss = F.ctc_loss(lp, targets, input_lengths, target_lengths, blank=self.blank, reduction="sum",
                          zero_infinity=self.zero_infinity)
        if self.label_smoothing > 0:
            T, B, V = lp.shape
            valid = (torch.arange(T, device=lp.device)[:, None] < input_lengths[None, :]).unsqueeze(-1)
            kl = -(lp * valid).sum() / V
            loss = (1 - self.label_smoothing) * loss + self.label_smoothing * kl
        return loss, int(target_lengths.sum())


CTC = CTCLossFunc


class NMTAndCTCLossFunc(nn.Module):
    def __init__(self, hidden_size, output_size, label_smoothing=0.0, ctc_weight=0.3, padding_idx=0):
        super().__init__()
        self.nmt = NMTLossFunc(hidden_size, output_size, label_smoothing, padding_idx=padding_idx)
        self.ctc = CTCLossFunc(output_size, padding_idx=padding_idx)
        self.ctc_weight = ctc_weight

    def forward(self, model_outputs, targets, **kw):
        out = self.nmt(model_outputs, targets)
        if "encoder_logits" in model_outputs:
            ctc, n = self.ctc(model_outputs["encoder_logits"], model_outputs["src_lengths"], kw["ctc_targets"])
            out["ctc_loss"], out["n_ctc_targets"] = ctc, n
            out["loss"] = (1 - self.ctc_weight) * out["loss"] + self.ctc_weight * ctc
        return out


class MPCLoss(nn.Module):
    """L1 reconstruction of masked input frames (masked predictive coding)."""

    def forward(self, model_outputs):
        pred, target, mask = model_outputs["mpc"], model_outputs["original_source"], model_outputs["masked_positions"]
        diff = (pred.float() - target.float()).abs() * mask.unsqueeze(-1)
        loss = diff.sum()
        return {"loss": loss, "data": float(loss.detach()), "numel": int(mask.sum()) * pred.shape[-1]}


class ClassifierLoss(nn.Module):
    def __init__(self, hidden_size: int, output_size: int, label_smoothing: float = 0.0):
        super().__init__()
        self.label_smoothing = label_smoothing

    def forward(self, model_outputs, targets, mask=None):
        logits = model_outputs["logits"].float()
        flat, tgt = logits.reshape(-1, logits.shape[-1]), targets.reshape(-1)
        loss = F.cross_entropy(flat, tgt, reduction="none", label_smoothing=self.label_smoothing if self.training else 0.0)
        if mask is not None:
            keep = ~mask.reshape(-1)
            loss = loss * keep
            n = int(keep.sum())
        else:
            n = tgt.numel()
        correct = int(((flat.argmax(-1) == tgt) & (keep if mask is not None else torch.ones_like(tgt, dtype=torch.bool))).sum())
        return {"loss": loss.sum(), "data": float(loss.detach().sum()), "numel": n, "n_correct": correct}


class CrossEntropyLIDLoss(nn.Module):
    """Per-frame language-id cross-entropy over encoder states; ``targets`` is one label per utterance."""

    def __init__(self, output_size: int, label_smoothing: float = 0.0):
        super().__init__()
        self.label_smoothing = label_smoothing

    def forward(self, lid_logits, targets, mask=None):
        T, B, V = lid_logits.shape
        tgt = targets.view(1, B).expand(T, B).reshape(-1)
        loss = F.cross_entropy(lid_logits.reshape(-1, V).float(), tgt, reduction="none", label_smoothing=self.label_smoothing)
        if mask is not None:
            loss = loss * (~mask.t().reshape(-1))
        return loss.sum()


def kl_distillation(student_logits, teacher_logits, mask=None, temperature: float = 1.0):
    """sum over positions of KL(teacher || student); used by dark-experience-replay style trainers."""
    s = F.log_softmax(student_logits.float() / temperature, -1)
    t = F.softmax(teacher_logits.float() / temperature, -1)
    kl = (t * (torch.log(t.clamp_min(1e-20)) - s)).sum(-1)
    if mask is not None:
        kl = kl * mask
    return kl.sum() * temperature * temperature
