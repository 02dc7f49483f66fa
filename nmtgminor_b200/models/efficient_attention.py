"""Sub-quadratic and latent attention variants kept for the research model families: FAVOR+ (Performer) random-feature
attention, LSH bucketed attention, a Perceiver-style latent bottleneck, and MaxOut.

All operate on padded ``[B, T, H]`` tensors with a boolean ``key_padding_mask`` (True = pad).

Reference: onmt/modules/performer.py (``FastAttention``, ``softmax_kernel``, ``gaussian_orthogonal_random_matrix``),
onmt/modules/lsh_attention.py, onmt/models/speech_recognizer/perceiver/, onmt/modules/linear.py (``MaxOut``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


def gaussian_orthogonal_random_matrix(rows: int, cols: int, generator=None) -> torch.Tensor:
    """Blocks of orthogonal directions rescaled to the norms of Gaussian vectors (lower-variance random features)."""
    blocks = []
    for _ in range(math.ceil(rows / cols)):
        q, _ = torch.linalg.qr(torch.randn(cols, cols, generator=generator))
        blocks.append(q.t())
    m = torch.cat(blocks, 0)[:rows]
    norms = torch.randn(rows, cols, generator=generator).norm(dim=1)
    return norms[:, None] * m


def softmax_kernel(x, projection, is_query: bool, eps: float = 1e-4):
    """Positive random features whose inner products estimate ``exp(q . k)`` (FAVOR+)."""
    d = x.shape[-1]
    x = x * d ** -0.25
    proj = x @ projection.t().to(x.dtype)
    sq = (x ** 2).sum(-1, keepdim=True) / 2
    stab = proj.amax(dim=-1, keepdim=True) if is_query else proj.amax(dim=(-1, -2), keepdim=True)
    return (torch.exp(proj - sq - stab) + eps) * projection.shape[0] ** -0.5


class PerformerAttention(nn.Module):
    """Linear-time multi-head attention through random features; ``causal`` uses prefix sums."""

    def __init__(self, dim: int, heads: int, nb_features: Optional[int] = None, causal: bool = False, seed: int = 0):
        super().__init__()
        self.heads, self.hd, self.causal = heads, dim // heads, causal
        self.qkv, self.out = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        m = nb_features or int(self.hd * math.log(self.hd))
        self.register_buffer("projection", gaussian_orthogonal_random_matrix(m, self.hd, torch.Generator().manual_seed(seed)))

    def forward(self, x, key_padding_mask=None):
        B, T, H = x.shape
        q, k, v = self.qkv(x).view(B, T, 3, self.heads, self.hd).permute(2, 0, 3, 1, 4)      # [B, h, T, d]
        qf, kf = softmax_kernel(q.float(), self.projection, True), softmax_kernel(k.float(), self.projection, False)
        v = v.float()
        if key_padding_mask is not None:
            keep = (~key_padding_mask)[:, None, :, None].float()
            kf, v = kf * keep, v * keep
        if self.causal:
            kv = torch.cumsum(torch.einsum("bhtm,bhtd->bhtmd", kf, v), 2)
            z = torch.cumsum(kf, 2)
            num = torch.einsum("bhtm,bhtmd->bhtd", qf, kv)
            den = torch.einsum("bhtm,bhtm->bht", qf, z)
        else:
            kv = torch.einsum("bhtm,bhtd->bhmd", kf, v)
            num = torch.einsum("bhtm,bhmd->bhtd", qf, kv)
            den = torch.einsum("bhtm,bhm->bht", qf, kf.sum(2))
        ctx = (num / den.clamp_min(1e-6)[..., None]).transpose(1, 2).reshape(B, T, H)
        return self.out(ctx.to(x.dtype))


class LSHAttention(nn.Module):
    """Attention restricted to keys that fall into the same random-rotation hash bucket as the query (shared QK),
    over ``rounds`` independent hashes whose results are averaged; every token always attends to itself."""

    def __init__(self, dim: int, heads: int, buckets: int = 8, rounds: int = 2, seed: int = 0):
        super().__init__()
        self.heads, self.hd, self.buckets, self.rounds = heads, dim // heads, buckets, rounds
        self.qk, self.v, self.out = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
        g = torch.Generator().manual_seed(seed)
        self.register_buffer("rotations", torch.randn(rounds, self.hd, buckets // 2, generator=g))

    def forward(self, x, key_padding_mask=None):
        B, T, H = x.shape
        qk = self.qk(x).view(B, T, self.heads, self.hd).transpose(1, 2).float()
        v = self.v(x).view(B, T, self.heads, self.hd).transpose(1, 2).float()
        unit = F.normalize(qk, dim=-1)
        outs = 0
        for r in range(self.rounds):
            rot = unit @ self.rotations[r]
            bucket = torch.cat([rot, -rot], -1).argmax(-1)                    # [B, h, T]
            same = bucket[..., :, None] == bucket[..., None, :]
            same = same | torch.eye(T, dtype=torch.bool, device=x.device)
            s = (qk @ unit.transpose(-1, -2)) * self.hd ** -0.5
            s = s.masked_fill(~same, float("-inf"))
            if key_padding_mask is not None:
                s = s.masked_fill(key_padding_mask[:, None, None, :] & ~torch.eye(T, dtype=torch.bool, device=x.device), float("-inf"))
            outs = outs + torch.softmax(s, -1) @ v
        ctx = (outs / self.rounds).transpose(1, 2).reshape(B, T, H)
        return self.out(ctx.to(x.dtype))


class PerceiverBottleneck(nn.Module):
    """``n_latents`` learned queries cross-attend to the (long) input, are refined by self-attention blocks, and
    replace the input as a fixed-length memory for the decoder."""

    def __init__(self, dim: int, heads: int, n_latents: int = 64, layers: int = 2, dropout: float = 0.0):
        super().__init__()
        self.latents = nn.Parameter(torch.randn(n_latents, dim) * dim ** -0.5)
        self.cross = nn.MultiheadAttention(dim, heads, dropout=dropout, batch_first=True)
        self.cross_norm, self.in_norm = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.blocks = nn.ModuleList([nn.TransformerEncoderLayer(dim, heads, 4 * dim, dropout, batch_first=True, norm_first=True)
                                     for _ in range(layers)])
        self.out_norm = nn.LayerNorm(dim)

    def forward(self, x, key_padding_mask=None):
        B = x.shape[0]
        lat = self.latents[None].expand(B, -1, -1)
        att, _ = self.cross(self.cross_norm(lat), self.in_norm(x), self.in_norm(x), key_padding_mask=key_padding_mask, need_weights=False)
        lat = lat + att
        for blk in self.blocks:
            lat = blk(lat)
        return self.out_norm(lat)


class MaxOut(nn.Module):
    """Linear layer with ``pool`` candidates per output unit, of which the maximum is kept."""

    def __init__(self, in_dim: int, out_dim: int, pool: int = 2):
        super().__init__()
        self.lin, self.out_dim, self.pool = nn.Linear(in_dim, out_dim * pool), out_dim, pool

    def forward(self, x):
        return self.lin(x).view(*x.shape[:-1], self.out_dim, self.pool).amax(-1)


def apply_chunking_to_forward(chunk_size: int, chunk_dim: int, forward_fn, *tensors):
    """Runs ``forward_fn`` on slices of ``chunk_size`` along ``chunk_dim`` and concatenates the results: the same output
    as one call when ``forward_fn`` treats positions along that dimension independently (a feed-forward block), with the
    intermediate activations of one slice alive at a time.  ``chunk_size`` 0 = one call.
    Reference: onmt/legacy/old_models/reformer.py:28-84."""
    assert tensors and all(t.shape == tensors[0].shape for t in tensors), "inputs must share one shape"
    if chunk_size <= 0 or tensors[0].shape[chunk_dim] <= chunk_size:
        return forward_fn(*tensors)
    pieces = zip(*(t.split(chunk_size, dim=chunk_dim) for t in tensors))      # the last slice may be shorter
    return torch.cat([forward_fn(*piece) for piece in pieces], dim=chunk_dim)


class ReformerEncoderLayer(nn.Module):
    """Pre-norm encoder layer with bucketed (LSH) self-attention and a feed-forward block evaluated in slices along the
    time axis; stochastic depth with probability ``death_rate`` (outputs rescaled by ``1 / (1 - death_rate)`` when kept).
    Reference: onmt/legacy/old_models/reformer.py:87-129 (``ReformerEncoderLayer``)."""

    def __init__(self, dim: int, heads: int, inner: int, dropout: float = 0.1, death_rate: float = 0.0, buckets: int = 8,
                 rounds: int = 2, ffn_chunk: int = 0, seed: int = 0):
        super().__init__()
        self.attn_norm, self.ffn_norm = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.self_attention = LSHAttention(dim, heads, buckets, rounds, seed)
        self.fc1, self.fc2 = nn.Linear(dim, inner), nn.Linear(inner, dim)
        self.dropout, self.death_rate, self.ffn_chunk = dropout, death_rate, ffn_chunk

    def _ffn(self, x):
        return self.fc2(F.dropout(F.relu(self.fc1(x)), self.dropout, self.training))

    def forward(self, x, key_padding_mask=None):                  # x [B, T, H]
        if self.training and self.death_rate > 0 and torch.rand(()).item() < self.death_rate:
            return x
        keep = 1.0 / (1.0 - self.death_rate) if (self.training and self.death_rate > 0) else 1.0
        a = self.self_attention(self.attn_norm(x), key_padding_mask)
        x = x + F.dropout(a, self.dropout, self.training) * keep
        f = apply_chunking_to_forward(self.ffn_chunk, 1, self._ffn, self.ffn_norm(x))
        return x + F.dropout(f, self.dropout, self.training) * keep
