"""Pluggable scaled-dot-product attention for the typed building blocks: every ``StandardMultiheadAttention`` owns an
``SDPA`` object that turns projected queries / keys / values ``[B, heads, T, d]`` into context vectors (and, on request,
attention weights); which class is created by default is a process-wide, context-manageable choice.

* ``TorchSDPA``                  - PyTorch's fused attention (no weights returned);
* ``NaiveSDPA``                  - the explicit softmax, for attention-weight hooks and as the oracle in tests;
* ``RelativePositionSDPA``       - Transformer-XL style: content scores ``(q + u) k^T`` plus position scores
                                   ``(q + v) r^T`` shifted so that column j of row i holds the encoding of offset ``i - j``;
* ``ShawRelativePositionSDPA``   - clipped relative-position embeddings added to the keys (and optionally the values);
* ``AttentionWeightStoreHook``   - collects the weights of the layers it is registered on;
* ``ModuleList``                 - layer list with LayerDrop (each layer skipped with probability ``drop_p`` in training).

Reference: onmt/nn/transformer/attention.py:30-790 (``SDPA`` :30, ``TorchSDPA`` :86, ``NaiveSDPA`` :196,
``RelativePositionSDPA`` :284, ``RelativePositionalEncoding`` :454, ``ShawRelativePositionSDPA`` :561, factory :749-790),
onmt/nn/transformer/multihead_attention.py:117-160 (weight hooks), onmt/nn/module_list.py:17-80.
"""
from __future__ import annotations

import math
from contextlib import contextmanager
from typing import Callable, Iterator, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class SDPA(nn.Module):
    """``forward(q, k, v, mask, needs_weights) -> (context [B, h, Tq, d], weights [B, h, Tq, Tk] or None)``; ``mask`` is
    an additive float mask broadcastable to ``[B, h, Tq, Tk]``."""

    def __init__(self, attn_dropout_p: float = 0.0):
        super().__init__()
        self.attn_dropout_p = attn_dropout_p

    def forward(self, q, k, v, mask=None, needs_weights: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError


def _naive(q, scores, v, mask, dropout_p, training, needs_weights):
    if mask is not None:
        scores = scores + mask.to(scores.dtype)
    w = torch.softmax(scores.float(), dim=-1).to(q.dtype)
    w = torch.nan_to_num(w, nan=0.0)
    wd = F.dropout(w, dropout_p, training) if dropout_p > 0 else w
    return torch.matmul(wd, v), (w if needs_weights else None)


class TorchSDPA(SDPA):
    def forward(self, q, k, v, mask=None, needs_weights: bool = False):
        if needs_weights:
            return NaiveSDPA.forward(self, q, k, v, mask, True)
        p = self.attn_dropout_p if self.training else 0.0
        return F.scaled_dot_product_attention(q, k, v, attn_mask=None if mask is None else mask.to(q.dtype), dropout_p=p), None


class NaiveSDPA(SDPA):
    def forward(self, q, k, v, mask=None, needs_weights: bool = False):
        scores = torch.matmul(q, k.transpose(-1, -2)) * (q.shape[-1] ** -0.5)
        return _naive(q, scores, v, mask, self.attn_dropout_p, self.training, needs_weights)


class RelativePositionalEncoding(nn.Module):
    """Sinusoidal encodings of the offsets ``T-1 .. -(T-1)`` (``[2T - 1, dim]``), cached and grown on demand."""

    def __init__(self, encoding_dim: int, max_seq_len: int = 512):
        super().__init__()
        if encoding_dim % 2:
            raise ValueError("the encoding dimension must be even")
        self.encoding_dim = encoding_dim
        self.register_buffer("freqs", self._table(max_seq_len), persistent=False)

    def _table(self, T: int) -> torch.Tensor:
        offsets = torch.arange(T - 1, -T, -1, dtype=torch.float32)[:, None]        # T-1 .. -(T-1)
        inv = torch.exp(torch.arange(0, self.encoding_dim, 2, dtype=torch.float32) * (-math.log(10000.0) / self.encoding_dim))
        t = torch.zeros(2 * T - 1, self.encoding_dim)
        t[:, 0::2], t[:, 1::2] = torch.sin(offsets * inv), torch.cos(offsets * inv)
        return t

    def forward(self, seq_len: int, device=None) -> torch.Tensor:
        T = (self.freqs.shape[0] + 1) // 2
        if seq_len > T:
            self.freqs = self._table(seq_len).to(self.freqs.device)
            T = seq_len
        out = self.freqs[T - seq_len: T + seq_len - 1]
        return out.to(device) if device is not None else out


class RelativePositionSDPA(SDPA):
    """Self-attention scores ``(q + u) k^T + shift((q + v) (W_r r)^T)`` (Dai et al., 2019), one ``u`` / ``v`` bias per head."""

    def __init__(self, model_dim: int, num_heads: int, pos_encoding: Optional[RelativePositionalEncoding] = None,
                 attn_dropout_p: float = 0.0):
        super().__init__(attn_dropout_p)
        self.num_heads, self.head_dim = num_heads, model_dim // num_heads
        self.pos_encoding = pos_encoding or RelativePositionalEncoding(model_dim)
        self.r_proj = nn.Linear(model_dim, model_dim, bias=False)
        self.u_bias = nn.Parameter(torch.zeros(num_heads, self.head_dim))
        self.v_bias = nn.Parameter(torch.zeros(num_heads, self.head_dim))
        nn.init.xavier_normal_(self.u_bias)
        nn.init.xavier_normal_(self.v_bias)

    @staticmethod
    def _shift(x: torch.Tensor) -> torch.Tensor:
        """``[B, h, T, 2T - 1]`` indexed by offset ``T-1 .. -(T-1)`` -> ``[B, h, T, T]`` indexed by key position:
        ``out[i, j] = x[i, j + T - 1 - i]``, the entry of offset ``i - j``."""
        B, h, T, _ = x.shape
        x = F.pad(x, (1, 0))                                   # [B, h, T, 2T]
        x = x.view(B, h, 2 * T, T)[:, :, 1:].reshape(B, h, T, 2 * T - 1)
        return x[..., :T]

    def forward(self, q, k, v, mask=None, needs_weights: bool = False):
        if q.shape[2] != k.shape[2]:
            raise ValueError("relative-position attention is defined for self-attention (equal query and key lengths)")
        T = q.shape[2]
        r = self.r_proj(self.pos_encoding(T, q.device).to(q.dtype)).view(2 * T - 1, self.num_heads, self.head_dim).transpose(0, 1)
        ac = torch.matmul(q + self.u_bias[None, :, None, :].to(q.dtype), k.transpose(-1, -2))
        bd = self._shift(torch.matmul(q + self.v_bias[None, :, None, :].to(q.dtype), r.transpose(-1, -2)[None]))
        scores = (ac + bd) * (self.head_dim ** -0.5)
        return _naive(q, scores, v, mask, self.attn_dropout_p, self.training, needs_weights)


class ShawRelativePositionSDPA(SDPA):
    """Scores ``q (k + r_k[clip(j - i)])^T``; with ``use_rel_pos_values`` also ``sum_j w_ij (v_j + r_v[clip(j - i)])``
    (Shaw et al., 2018).  Offsets are clipped to ``[-max_left, max_right]`` (``max_right`` defaults to ``max_left``)."""

    def __init__(self, model_dim: int, num_heads: int, max_left_rel_pos: int, max_right_rel_pos: Optional[int] = None,
                 use_rel_pos_values: bool = False, attn_dropout_p: float = 0.0):
        super().__init__(attn_dropout_p)
        self.head_dim = model_dim // num_heads
        self.max_left = max_left_rel_pos
        self.max_right = max_left_rel_pos if max_right_rel_pos is None else max_right_rel_pos
        n = self.max_left + self.max_right + 1
        self.rel_k_embed = nn.Embedding(n, self.head_dim)
        self.rel_v_embed = nn.Embedding(n, self.head_dim) if use_rel_pos_values else None
        init_shaw_embedding(self.rel_k_embed)
        if self.rel_v_embed is not None:
            init_shaw_embedding(self.rel_v_embed)

    def rel_indices(self, q_len: int, k_len: int, device) -> torch.Tensor:
        i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
        j = torch.arange(k_len, device=device)[None, :]
        return (j - i).clamp(-self.max_left, self.max_right) + self.max_left

    def forward(self, q, k, v, mask=None, needs_weights: bool = False):
        idx = self.rel_indices(q.shape[2], k.shape[2], q.device)                 # [Tq, Tk]
        scores = torch.matmul(q, k.transpose(-1, -2))
        rk = self.rel_k_embed(idx).to(q.dtype)                                   # [Tq, Tk, d]
        scores = (scores + torch.einsum("bhqd,qkd->bhqk", q, rk)) * (self.head_dim ** -0.5)
        if mask is not None:
            scores = scores + mask.to(scores.dtype)
        w = torch.nan_to_num(torch.softmax(scores.float(), -1).to(q.dtype), nan=0.0)
        wd = F.dropout(w, self.attn_dropout_p, self.training) if self.attn_dropout_p > 0 else w
        ctx = torch.matmul(wd, v)
        if self.rel_v_embed is not None:
            ctx = ctx + torch.einsum("bhqk,qkd->bhqd", wd, self.rel_v_embed(idx).to(q.dtype))
        return ctx, (w if needs_weights else None)


def init_shaw_embedding(embed: nn.Embedding) -> None:
    nn.init.xavier_uniform_(embed.weight)


# ---- default factory -----------------------------------------------------------------------------------------
SDPAFactory = Callable[..., SDPA]
_default_factory: List[Optional[SDPAFactory]] = [None]


def set_default_sdpa_factory(factory: Optional[SDPAFactory]) -> None:
    """``factory(attn_dropout_p=...) -> SDPA`` used by attention modules that are not given an ``sdpa``; ``None`` restores
    ``TorchSDPA``."""
    _default_factory[0] = factory


def create_default_sdpa(*, attn_dropout_p: float = 0.0) -> SDPA:
    f = _default_factory[0] or TorchSDPA
    return f(attn_dropout_p=attn_dropout_p)


@contextmanager
def default_sdpa_factory(factory: Optional[SDPAFactory]) -> Iterator[None]:
    prev = _default_factory[0]
    _default_factory[0] = factory
    try:
        yield
    finally:
        _default_factory[0] = prev


# ---- attention-weight hooks ------------------------------------------------------------------------------------
class AttentionWeightStoreHook:
    """Callable ``hook(module, attn, attn_weights)`` that appends ``(attn, attn_weights)`` to ``storage``."""

    def __init__(self, storage: Optional[list] = None):
        self.storage = storage if storage is not None else []

    def __call__(self, module, attn, attn_weights) -> None:
        self.storage.append((attn, attn_weights))


# ---- layer list with LayerDrop -----------------------------------------------------------------------------------
class ModuleList(nn.ModuleList):
    """``drop_iter()`` yields the layers, each skipped with probability ``drop_p`` while training (never in evaluation)."""

    def __init__(self, modules=None, *, drop_p: float = 0.0):
        super().__init__(modules)
        self.drop_p = drop_p

    def drop_iter(self, generator: Optional[torch.Generator] = None) -> Iterator[nn.Module]:
        if self.drop_p > 0.0 and self.training:
            keep = torch.rand(len(self), generator=generator) > self.drop_p
        else:
            keep = None
        for i, m in enumerate(super().__iter__()):
            if keep is None or bool(keep[i]):
                yield m

    def extra_repr(self) -> str:
        return "drop_p=%g" % self.drop_p
