"""Jamba building blocks: grouped-query causal attention without positional encoding, RMS normalisation, the top-k
mixture-of-experts feed-forward block and the router load-balancing loss.

The reference keeps three pieces of the Jamba model (``onmt/models/jamba/jamba_attention.py:4-96`` eager attention,
``:97-373`` unpadded flash variant, ``:375-456`` SDPA variant; ``onmt/models/jamba/rms_norm.py:32-50``;
``onmt/models/jamba/load_balancing_loss.py:32-111``).  Here there is one attention class: it packs the valid tokens,
repeats the key / value heads up to the number of query heads and calls the packed causal attention of this library
(tensor-core kernels on a GPU for head sizes up to 64, the PyTorch statement elsewhere), so the "eager", "flash" and
"sdpa" variants collapse into the dispatch of ``ops.self_attention``.  Parameter names follow the published checkpoints
(``q_proj / k_proj / v_proj / o_proj``, ``weight`` of the norm, ``router`` / ``experts.N.{gate,up,down}_proj``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class JambaRMSNorm(nn.Module):
    """``x / sqrt(mean(x^2) + eps) * weight`` computed in fp32 and returned in the input's dtype."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x):
        x32 = x.float()
        y = x32 * torch.rsqrt(x32.square().mean(-1, keepdim=True) + self.variance_epsilon)
        return (self.weight.float() * y).to(x.dtype)


class KVCache:
    """Keys and values of the tokens seen so far, per layer: ``update`` appends along time and returns the full tensors
    (the attention part of the reference's hybrid cache; the state-space part belongs to layers this module does not
    have)."""

    def __init__(self):
        self.k: dict = {}
        self.v: dict = {}

    def update(self, k, v, layer_idx: int):
        if layer_idx in self.k:
            k = torch.cat([self.k[layer_idx], k], 1)
            v = torch.cat([self.v[layer_idx], v], 1)
        self.k[layer_idx], self.v[layer_idx] = k, v
        return k, v

    def seen(self, layer_idx: int) -> int:
        return 0 if layer_idx not in self.k else self.k[layer_idx].shape[1]


class JambaAttention(nn.Module):
    """Causal grouped-query attention: ``heads`` query heads share ``kv_heads`` key / value heads; no bias, no positional
    term (the state-space layers of the full model carry position)."""

    def __init__(self, hidden_size: int, heads: int, kv_heads: Optional[int] = None, attention_dropout: float = 0.0,
                 layer_idx: int = 0):
        super().__init__()
        kv_heads = kv_heads or heads
        if hidden_size % heads or heads % kv_heads:
            raise ValueError("hidden_size must be divisible by heads, and heads by kv_heads (got %d, %d, %d)"
                             % (hidden_size, heads, kv_heads))
        self.hidden_size, self.num_heads, self.num_key_value_heads = hidden_size, heads, kv_heads
        self.head_dim = hidden_size // heads
        self.num_key_value_groups = heads // kv_heads
        self.attention_dropout = attention_dropout
        self.layer_idx = layer_idx
        self.q_proj = nn.Linear(hidden_size, heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, kv_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, kv_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(heads * self.head_dim, hidden_size, bias=False)

    def _repeat(self, t):
        """[..., kv_heads * d] -> [..., heads * d]: query head ``h`` reads key / value head ``h // groups``."""
        if self.num_key_value_groups == 1:
            return t
        lead = t.shape[:-1]
        t = t.reshape(*lead, self.num_key_value_heads, 1, self.head_dim)
        return t.expand(*lead, self.num_key_value_heads, self.num_key_value_groups, self.head_dim).reshape(*lead, -1)

    def forward(self, hidden_states, lengths: Optional[torch.Tensor] = None, cache: Optional[KVCache] = None):
        """``hidden_states [B, T, H]``; ``lengths [B]`` marks right-padded rows (their outputs are zero).  With ``cache``
        the new tokens attend to everything stored for this layer plus themselves (incremental decoding; no padding)."""
        B, T, _ = hidden_states.shape
        q = self.q_proj(hidden_states)
        k = self.k_proj(hidden_states)
        v = self.v_proj(hidden_states)
        if cache is not None:
            past = cache.seen(self.layer_idx)
            k, v = cache.update(k, v, self.layer_idx)
            Tk = k.shape[1]
            qh = q.view(B, T, self.num_heads, self.head_dim).transpose(1, 2)
            kh = self._repeat(k).view(B, Tk, self.num_heads, self.head_dim).transpose(1, 2)
            vh = self._repeat(v).view(B, Tk, self.num_heads, self.head_dim).transpose(1, 2)
            allowed = (torch.arange(Tk, device=q.device)[None, :] <= past + torch.arange(T, device=q.device)[:, None])
            ctx = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=allowed[None, None])
            return self.o_proj(ctx.transpose(1, 2).reshape(B, T, -1))
        if lengths is None:
            lengths = torch.full((B,), T, dtype=torch.int64, device=hidden_states.device)
        valid = (torch.arange(T, device=hidden_states.device)[None, :] < lengths[:, None]).reshape(-1)
        rows = valid.nonzero(as_tuple=False).squeeze(1)
        qkv = torch.cat([q, self._repeat(k), self._repeat(v)], -1).reshape(B * T, -1).index_select(0, rows)
        cu = torch.zeros(B + 1, dtype=torch.int32, device=hidden_states.device)
        cu[1:] = lengths.cumsum(0)
        ctx = ops.self_attention(qkv, cu, self.num_heads, T, causal=True, dropout_p=self.attention_dropout, training=self.training)
        out = self.o_proj(ctx)
        full = out.new_zeros(B * T, self.hidden_size)
        return full.index_copy(0, rows, out).view(B, T, self.hidden_size)


class JambaMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class JambaSparseMoeBlock(nn.Module):
    """Top-k routed experts: every token is sent to its ``top_k`` experts (softmax over all experts, weights of the chosen
    ones kept without renormalisation) and the expert outputs are summed with those weights.  Returns the mixed output
    and the router logits ``[tokens, experts]`` that the load-balancing loss wants."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int = 2):
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k
        self.router = nn.Linear(hidden_size, num_experts, bias=False)
        self.experts = nn.ModuleList(JambaMLP(hidden_size, intermediate_size) for _ in range(num_experts))

    def forward(self, x) -> Tuple[torch.Tensor, torch.Tensor]:
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        logits = self.router(flat)
        weights, chosen = torch.softmax(logits.float(), -1).topk(self.top_k, -1)
        out = torch.zeros_like(flat)
        for e, expert in enumerate(self.experts):
            token, slot = (chosen == e).nonzero(as_tuple=True)
            if token.numel():
                out.index_add_(0, token, expert(flat.index_select(0, token)) * weights[token, slot, None].to(flat.dtype))
        return out.view(shape), logits


def load_balancing_loss(router_logits: Optional[Sequence[torch.Tensor]], num_experts: int, top_k: int = 2,
                        attention_mask: Optional[torch.Tensor] = None):
    """Switch-Transformer auxiliary loss over all routed layers: ``num_experts * sum_e f_e * P_e`` where ``f_e`` is the
    fraction of (token, slot) assignments that went to expert ``e`` (per slot of the top-k) and ``P_e`` the mean router
    probability of ``e``.  ``router_logits``: one ``[batch * time, experts]`` tensor per layer; ``attention_mask
    [batch, time]`` (1 = real token) leaves padding out of both means.  Returns 0 when there is nothing to balance."""
    if router_logits is None or not isinstance(router_logits, (tuple, list)) or len(router_logits) == 0:
        return 0
    logits = torch.cat([l.float() for l in router_logits], 0)             # [layers * tokens, E]
    probs = torch.softmax(logits, -1)
    _, chosen = probs.topk(top_k, -1)
    assigned = F.one_hot(chosen, num_experts).float()                     # [layers * tokens, k, E]
    if attention_mask is None:
        tokens_per_expert = assigned.mean(0)                              # [k, E]
        prob_per_expert = probs.mean(0)                                   # [E]
    else:
        layers = logits.shape[0] // attention_mask.numel()
        w = attention_mask.reshape(-1).float().repeat(layers)             # [layers * tokens]
        tokens_per_expert = (assigned * w[:, None, None]).sum(0) / w.sum().clamp_min(1.0)
        prob_per_expert = (probs * w[:, None]).sum(0) / w.sum().clamp_min(1.0)
    return (tokens_per_expert * prob_per_expert[None]).sum() * num_experts


class JambaAttentionDecoderLayer(nn.Module):
    """Pre-norm attention layer of the hybrid stack: RMSNorm -> attention -> residual, RMSNorm -> dense MLP or routed
    experts -> residual.  Returns ``(hidden, router_logits or None)``."""

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, intermediate_size: int, num_experts: int = 1,
                 top_k: int = 2, eps: float = 1e-6, attention_dropout: float = 0.0, layer_idx: int = 0):
        super().__init__()
        self.self_attn = JambaAttention(hidden_size, heads, kv_heads, attention_dropout, layer_idx)
        self.feed_forward = (JambaSparseMoeBlock(hidden_size, intermediate_size, num_experts, top_k) if num_experts > 1
                             else JambaMLP(hidden_size, intermediate_size))
        self.input_layernorm = JambaRMSNorm(hidden_size, eps)
        self.pre_ff_layernorm = JambaRMSNorm(hidden_size, eps)

    def forward(self, x, lengths=None, cache: Optional[KVCache] = None):
        x = x + self.self_attn(self.input_layernorm(x), lengths, cache)
        y = self.feed_forward(self.pre_ff_layernorm(x))
        logits = None
        if isinstance(y, tuple):
            y, logits = y
        return x + y, logits
