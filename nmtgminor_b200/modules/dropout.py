"""Dropout family beyond the element-wise dropout that the fused kernels regenerate from counters.

* ``VariationalDropout`` / ``variational_dropout``: one mask per sequence and feature, shared by all time steps
  (padded ``[T, B, H]`` / ``[B, T, H]`` tensors, or packed ``[N, H]`` rows with ``cu`` sentence boundaries);
* ``embedded_dropout`` / ``word_dropout_tokens``: drops whole vocabulary entries for one batch;
* ``switchout``: replaces a sampled number of words per sentence by random words;
* ``ReLUDropout`` / ``relu_dropout``: ReLU followed by (optionally variational) dropout;
* ``StaticDropout``: a mask that is sampled once and replayed (recomputation under activation checkpointing);
* ``checkpointed``: activation checkpointing that replays the counter-based dropout streams of the fused ops.

Reference: onmt/modules/dropout.py:8-160 (variational :8/:33, embedded :51, switchout :75, ReLU dropout :137/:150),
onmt/modules/static_dropout.py, onmt/modules/checkpoint.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from .. import constants as C


def _sentence_of_row(cu, n_rows: int):
    """Sentence index of every packed row (rows past ``cu[-1]``, the static padding, map to the last sentence)."""
    B = cu.numel() - 1
    pos = torch.arange(n_rows, device=cu.device, dtype=cu.dtype)
    return torch.bucketize(pos, cu[1:].contiguous(), right=True).clamp_(max=B - 1)


def variational_dropout(x, p: float = 0.5, training: bool = True, batch_first: bool = False, cu: Optional[torch.Tensor] = None):
    """Dropout whose mask is constant along time.  ``cu`` (int32 ``[B + 1]``) marks packed rows ``[N, H]``."""
    if not training or p <= 0:
        return x
    keep = 1.0 - p
    if cu is not None:
        B = cu.numel() - 1
        mask = torch.bernoulli(torch.full((B, x.shape[-1]), keep, device=x.device, dtype=torch.float32)) / keep
        rows = _sentence_of_row(cu, x.shape[0])
        return x * mask.to(x.dtype)[rows]
    if x.dim() == 3:
        shape = (x.shape[0], 1, x.shape[2]) if batch_first else (1, x.shape[1], x.shape[2])
    else:
        shape = x.shape
    mask = torch.bernoulli(torch.full(shape, keep, device=x.device, dtype=torch.float32)) / keep
    return x * mask.to(x.dtype)


class VariationalDropout(nn.Module):
    def __init__(self, p: float = 0.5, batch_first: bool = False):
        super().__init__()
        self.p, self.batch_first = p, batch_first

    def forward(self, x, cu=None):
        return variational_dropout(x, self.p, self.training, self.batch_first, cu)


def word_dropout_tokens(tokens, vocab_size: int, p: float, pad_idx: int = C.PAD):
    """Vocabulary-level dropout as a token rewrite: every word type is dropped with probability ``p`` for the whole
    batch; its occurrences become ``pad_idx`` (whose embedding row is zero).  Returns ``(tokens, scale)`` where
    ``scale = 1 / (1 - p)`` must multiply the surviving embeddings."""
    if p <= 0:
        return tokens, 1.0
    dropped = torch.rand(vocab_size, device=tokens.device) < p
    return torch.where(dropped[tokens], torch.full_like(tokens, pad_idx), tokens), 1.0 / (1.0 - p)


def embedded_dropout(embed: nn.Embedding, words, dropout: float = 0.1, scale=None):
    """``F.embedding`` with rows of the weight matrix dropped (and the rest rescaled) for this call."""
    weight = embed.weight
    if dropout:
        mask = torch.bernoulli(torch.full((weight.shape[0], 1), 1 - dropout, device=weight.device, dtype=weight.dtype)) / (1 - dropout)
        weight = mask * weight
    if scale is not None:
        weight = scale * weight
    pad = embed.padding_idx if getattr(embed, "padding_idx", None) is not None else -1
    return F.embedding(words, weight, pad)


def switchout(words, vocab_size: int, tau: float = 1.0, transpose: bool = False, offset: int = 0, generator=None):
    """SwitchOut: per sentence sample how many words to corrupt (``P(k) ~ exp(-k * tau)`` over its real words), then
    corrupt each real word with probability ``k / length`` by adding a random offset modulo the vocabulary.
    ``words`` is ``[B, T]`` (``transpose``: ``[T, B]``); BOS / EOS / PAD and the first ``offset`` columns stay."""
    if transpose:
        words = words.t()
    head = None
    if offset > 0:
        head, words = words[:, :offset], words[:, offset:]
    special = (words == C.BOS) | (words == C.EOS) | (words == C.PAD)
    lengths = (~special).float().sum(1).clamp_min(1.0)
    B, T = words.shape
    logits = -torch.arange(T, device=words.device, dtype=torch.float32)[None, :].expand(B, T) * tau
    logits = logits.masked_fill(special, float("-inf"))
    all_special = special.all(1, keepdim=True)
    logits = torch.where(all_special, torch.zeros_like(logits), logits)
    k = torch.multinomial(torch.softmax(logits, 1), 1, generator=generator).squeeze(1).float()
    prob = (k / lengths)[:, None].expand(B, T).masked_fill(special, 0.0).clamp(0, 1)
    corrupt = torch.bernoulli(prob, generator=generator).bool()
    shift = torch.randint(1, max(vocab_size, 2), words.shape, device=words.device, generator=generator)
    out = torch.where(corrupt, (words + shift) % vocab_size, words)
    if head is not None:
        out = torch.cat([head, out], 1)
    return out.t() if transpose else out


def relu_dropout(x, p: float = 0.0, training: bool = False, variational: bool = False, batch_first: bool = False):
    x = F.relu(x)
    if not training or p <= 0:
        return x
    return variational_dropout(x, p, True, batch_first) if variational else F.dropout(x, p, True)


class ReLUDropout(nn.Dropout):
    def __init__(self, p: float = 0.5, variational: bool = False, batch_first: bool = False, inplace: bool = False):
        super().__init__(p, inplace)
        self.variational, self.batch_first = variational, batch_first

    def forward(self, x):
        return relu_dropout(x, self.p, self.training, self.variational, self.batch_first)


class StaticDropout(nn.Module):
    """Dropout with a replayable mask: ``sample_mask`` draws it, every ``forward`` until the next draw reuses it."""

    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p
        self.mask: Optional[torch.Tensor] = None

    def sample_mask(self, like):
        self.mask = torch.bernoulli(torch.full_like(like, 1 - self.p, dtype=torch.float32)).to(like.dtype) / (1 - self.p)
        return self.mask

    def forward(self, x, resample: bool = False):
        if not self.training or self.p <= 0:
            return x
        if resample or self.mask is None or self.mask.shape != x.shape:
            self.sample_mask(x)
        return x * self.mask


def checkpointed(fn, *args):
    """Activation checkpointing of ``fn(*args)``.  The fused ops derive their dropout masks from a per-step stream
    counter; the recomputation rewinds that counter to the value it had on entry, so it regenerates exactly the masks
    of the first pass (the role ``StaticDropout`` plays for stored masks)."""
    from .. import ops
    start = ops._Rng.counter
    state = {"first": True, "end": start}

    def run(*a):
        if state["first"]:
            state["first"] = False
            out = fn(*a)
            state["end"] = ops._Rng.counter
            return out
        saved = ops._Rng.counter
        ops._Rng.counter = start
        try:
            return fn(*a)
        finally:
            ops._Rng.counter = saved

    return _torch_checkpoint(run, *args, use_reentrant=False)


def switchout_packed(tokens, cu, vocab_size: int, tau: float = 1.0, generator=None):
    """``switchout`` for packed rows: ``tokens`` [N] with int32 sentence boundaries ``cu`` [B + 1]."""
    B = cu.numel() - 1
    lengths = (cu[1:] - cu[:-1]).long()
    rows = _sentence_of_row(cu, tokens.shape[0])
    special = (tokens == C.BOS) | (tokens == C.EOS) | (tokens == C.PAD)
    n_real = torch.zeros(B, device=tokens.device).scatter_add_(0, rows, (~special).float())
    t_max = int(lengths.max().item()) if B else 0
    ks = torch.arange(t_max, device=tokens.device, dtype=torch.float32)[None, :]
    logits = (-ks * tau).expand(B, t_max).masked_fill(ks >= n_real.clamp_min(1.0)[:, None], float("-inf"))
    k = torch.multinomial(torch.softmax(logits, 1), 1, generator=generator).squeeze(1).float()
    prob = (k / n_real.clamp_min(1.0))[rows].masked_fill(special, 0.0).clamp(0, 1)
    corrupt = torch.bernoulli(prob, generator=generator).bool()
    shift = torch.randint(1, max(vocab_size, 2), tokens.shape, device=tokens.device, generator=generator)
    return torch.where(corrupt, (tokens + shift) % vocab_size, tokens)
