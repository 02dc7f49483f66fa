"""Noise-contrastive estimation for large output vocabularies.

Instead of normalising over the whole vocabulary, every target word is scored against ``noise_ratio`` words drawn from a
fixed noise distribution (the unigram distribution of the training data) and the model learns to tell data from noise:
``P(data | w, h) = p_model(w | h) / (p_model(w | h) + k p_noise(w))`` with the partition function fixed to ``exp(logz)``.
Evaluation uses the ordinary softmax over the same weights.

* ``AliasSampler``  - O(1) draws from a fixed categorical distribution (Walker's alias method; the table is built once,
  in time linear in the vocabulary, with two work lists).
* ``build_unigram_noise`` - normalised word frequencies from a dictionary (or a uniform fallback).
* ``NCELinear`` - output layer: in training returns the scores of the target and of the shared noise sample plus
  their noise log-probabilities; in evaluation the full logits.
* ``NCELoss``   - the binary cross-entropy of data-vs-noise with label smoothing spread over the noise words.

Reference: onmt/modules/nce/nce_linear.py:12-232 (alias sampler :12, ``NCELinear`` :100), onmt/modules/nce/nce_loss.py:12-93,
onmt/modules/nce/nce_utils.py:1-23, model_factory.py:124-136.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

BACKOFF_PROB = 1e-10


class AliasSampler(nn.Module):
    """``draw(*size)`` returns int64 samples of the given shape from ``probs`` (must sum to 1)."""

    def __init__(self, probs: torch.Tensor):
        super().__init__()
        p = probs.detach().double().cpu()
        if abs(float(p.sum()) - 1.0) > 1e-4:
            raise ValueError("the noise distribution must sum to 1")
        K = p.numel()
        scaled = (p * K).tolist()
        alias = list(range(K))
        small = [i for i, x in enumerate(scaled) if x < 1.0]
        large = [i for i, x in enumerate(scaled) if x >= 1.0]
        # pair every under-full cell with an over-full one; each pairing finalises one cell, so this is linear
        while small and large:
            s, l = small.pop(), large[-1]
            alias[s] = l
            scaled[l] = scaled[l] - (1.0 - scaled[s])
            if scaled[l] < 1.0:
                small.append(large.pop())
        for i in small + large:                      # numerical leftovers keep their own cell
            scaled[i] = 1.0
        self.register_buffer("prob", torch.tensor(scaled, dtype=torch.float32).clamp_(0.0, 1.0))
        self.register_buffer("alias", torch.tensor(alias, dtype=torch.long))

    def draw(self, *size) -> torch.Tensor:
        K = self.alias.numel()
        cell = torch.randint(0, K, size, device=self.alias.device)
        keep = torch.rand(size, device=self.alias.device) < self.prob[cell]
        return torch.where(keep, cell, self.alias[cell])


def build_unigram_noise(freq: Optional[torch.Tensor] = None, vocab_size: int = 0, dictionary=None) -> torch.Tensor:
    """Normalised word frequencies ``[V]`` with a small floor so that no word has probability 0.  ``dictionary`` may be a
    ``Dict`` with a ``frequencies`` map (index -> count)."""
    if freq is None and dictionary is not None and getattr(dictionary, "frequencies", None):
        V = dictionary.size()
        freq = torch.zeros(V)
        for idx, c in dictionary.frequencies.items():
            if 0 <= int(idx) < V:
                freq[int(idx)] = float(c)
    if freq is None:
        freq = torch.ones(vocab_size if vocab_size > 0 else dictionary.size())
    freq = freq.float().clamp(min=0)
    total = float(freq.sum())
    probs = freq / total if total > 0 else torch.full_like(freq, 1.0 / freq.numel())
    probs = probs + BACKOFF_PROB
    return probs / probs.sum()


class NCELinear(nn.Module):
    """Output projection scored against a noise sample that is shared by all rows of the batch."""

    def __init__(self, hidden_size: int, output_size: int, noise_distribution: torch.Tensor, noise_ratio: int = 64,
                 weight: Optional[nn.Parameter] = None, bias=True):
        super().__init__()
        self.hidden_size, self.output_size, self.noise_ratio = hidden_size, output_size, int(noise_ratio)
        self.weight = weight if weight is not None else nn.Parameter(torch.randn(output_size, hidden_size) * hidden_size ** -0.5)
        if isinstance(bias, nn.Parameter):
            self.bias = bias                                                         # shared with the evaluation-time generator
        else:
            self.bias = nn.Parameter(torch.zeros(output_size)) if bias else None
        self.sampler = AliasSampler(noise_distribution)
        self.register_buffer("logprob_noise", noise_distribution.float().log())

    def _score(self, hidden, words):
        """hidden [N, H], words [N, k] (or [k], shared) -> scores [N, k]"""
        if words.dim() == 1:
            s = hidden.float() @ self.weight.index_select(0, words).float().t()
            return s + self.bias.index_select(0, words).float() if self.bias is not None else s
        w = self.weight[words].float()                                             # [N, k, H]
        s = torch.einsum("nh,nkh->nk", hidden.float(), w)
        return s + self.bias[words].float() if self.bias is not None else s

    def forward(self, hidden: torch.Tensor, targets: Optional[torch.Tensor] = None) -> Dict:
        if not self.training or targets is None:
            return {"logits": F.linear(hidden, self.weight.to(hidden.dtype), None if self.bias is None else self.bias.to(hidden.dtype))}
        noise = self.sampler.draw(self.noise_ratio)                                  # [k], one sample for the batch
        tgt = targets.view(-1, 1)
        return {"scores_model_target": self._score(hidden, tgt),
                "scores_model_noise": self._score(hidden, noise),
                "logprob_noise_target": self.logprob_noise[tgt],
                "logprob_noise_noise": self.logprob_noise[noise][None, :].expand(hidden.shape[0], -1),
                "noise_samples": noise}


class NCELoss(nn.Module):
    """``forward(model_outputs, targets)`` with the dictionary produced by ``NCELinear`` (training) or with ``logprobs`` /
    ``logits`` (evaluation: plain cross-entropy).  Returns the reference's loss dictionary."""

    def __init__(self, hidden_size: int = 0, output_size: int = 0, noise_ratio: int = 64, logz: float = 8.0,
                 label_smoothing: float = 0.0, padding_idx: int = 0):
        super().__init__()
        self.noise_ratio, self.logz, self.padding_idx = int(noise_ratio), float(logz), padding_idx
        self.label_smoothing = label_smoothing
        self.smoothing_value = label_smoothing / (self.noise_ratio + 1)
        self.confidence = 1.0 - label_smoothing

    def forward(self, model_outputs: Dict, targets: torch.Tensor, **_unused) -> Dict:
        gold = targets.reshape(-1)
        keep = (gold != self.padding_idx).nonzero(as_tuple=False).squeeze(1)
        if self.training and "scores_model_target" in model_outputs:
            pick = lambda k: model_outputs[k].float().index_select(0, keep)
            logit_model = torch.cat([pick("scores_model_target"), pick("scores_model_noise")], 1) - self.logz
            logit_noise = torch.cat([pick("logprob_noise_target"), pick("logprob_noise_noise")], 1)
            # log-odds of "this word came from the data": log p_model - log (k p_noise)
            logit_true = logit_model - logit_noise - math.log(self.noise_ratio)
            label = torch.full_like(logit_true, self.smoothing_value)
            label[:, 0] = self.confidence
            loss = F.binary_cross_entropy_with_logits(logit_true, label, reduction="sum")
        else:
            logits = model_outputs.get("logits", model_outputs.get("logprobs"))
            logits = logits.reshape(-1, logits.shape[-1]).float().index_select(0, keep)
            loss = F.cross_entropy(logits, gold.index_select(0, keep), reduction="sum")
        return {"loss": loss, "data": float(loss.detach()), "rev_loss": None, "rev_loss_data": None, "mirror_loss": None,
                "rec_loss": None, "rec_loss_data": None}
