"""Relative-position (Transformer-XL) self-attention on packed sequences.

``rel_self_attention(qkv, r, u, w, cu, heads, max_len, causal, p)`` computes, per sequence and head,
``softmax(((q + u) k^T + shift((q + w) r^T)) / sqrt(d)) v`` where ``r`` holds one projected position embedding per
distance (row ``center - d`` = distance ``d = i - j``).  CUDA tensors with sequences of at most 128 tokens run
``csrc/rel_attention.cu``; ``rel_self_attention_reference`` is the PyTorch statement of the same thing (CPU path and
test oracle).

Reference: onmt/modules/optimized/relative_self_attention_func.py (``RelativeSelfAttnFunc``) and its
``relative_self_attn_cuda`` extension.
"""
from __future__ import annotations

import torch

from . import _Rng, ext, next_stream


def rel_self_attention_reference(qkv, r, u, w, cu, heads: int, center: int, causal: bool = False):
    """fp32 PyTorch oracle (no dropout); returns ctx [N, H]."""
    N, H3 = qkv.shape
    H = H3 // 3
    d = H // heads
    out = torch.zeros(N, H, dtype=torch.float32, device=qkv.device)
    q, k, v = (t.float().view(N, heads, d) for t in (qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]))
    rr = r.float().view(-1, heads, d)
    uf, wf = u.float().view(heads, d), w.float().view(heads, d)
    for b in range(cu.numel() - 1):
        s0, s1 = int(cu[b]), int(cu[b + 1])
        T = s1 - s0
        if T <= 0:
            continue
        qi, ki, vi = q[s0:s1], k[s0:s1], v[s0:s1]
        ac = torch.einsum("ihd,jhd->hij", qi + uf, ki)
        dist = torch.arange(T, device=qkv.device)[:, None] - torch.arange(T, device=qkv.device)[None, :]
        rel = rr[center - dist]                                         # [T, T, heads, d]
        bd = torch.einsum("ihd,ijhd->hij", qi + wf, rel)
        s = (ac + bd) * d ** -0.5
        if causal:
            s = s.masked_fill(dist[None] < 0, float("-inf"))
        out[s0:s1] = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vi).reshape(T, H)
    return out


class _RelAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, r, u, w, cu, heads, max_len, center, causal, p, seed, stream):
        from . import LAUNCHES
        LAUNCHES[0] += 1
        scale = 64 ** -0.5
        out, lse = ext().rel_attn_fwd(qkv, r, u, w, cu, heads, max_len, center, causal, scale, p, seed, stream)
        ctx.save_for_backward(qkv, r, u, w, cu, lse)
        ctx.cfg = (heads, max_len, center, causal, scale, p, seed, stream)
        return out

    @staticmethod
    def backward(ctx, dctx):
        from . import LAUNCHES
        LAUNCHES[0] += 1
        qkv, r, u, w, cu, lse = ctx.saved_tensors
        heads, max_len, center, causal, scale, p, seed, stream = ctx.cfg
        dqkv, dr, du, dw = ext().rel_attn_bwd(qkv, r, u, w, cu, lse, dctx.contiguous(), heads, max_len, center, causal, scale, p, seed, stream)
        return (dqkv, dr.to(r.dtype), du, dw) + (None,) * 8


def rel_self_attention(qkv, r, u, w, cu, heads: int, max_len: int, center: int, causal: bool = False, p: float = 0.0,
                       training: bool = True):
    """qkv bf16 [N, 3H] (CUDA), r bf16 [L, H], u / w fp32 [heads, 64]; ``max_len`` <= 128."""
    p = p if training else 0.0
    return _RelAttnFn.apply(qkv.contiguous(), r.contiguous(), u.float().contiguous(), w.float().contiguous(), cu, heads, int(max_len),
                            int(center), bool(causal), float(p), _Rng.seed, next_stream() if p > 0 else 0)
