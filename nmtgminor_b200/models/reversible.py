"""Reversible Transformer layers: activations are recomputed from the layer outputs in backward, so a stack stores
two tensors regardless of depth.

The hidden state is a pair (x1, x2).  One layer computes ``y1 = x1 + F(x2)``, ``y2 = x2 + G(y1)`` with F the
self-attention (plus, in the decoder, the encoder-decoder attention) sub-layer and G the feed-forward sub-layer, both
pre-normalised.  Backward reconstructs ``x2 = y2 - G(y1)`` and ``x1 = y1 - F(x2)`` and differentiates the recomputed
sub-layers.  The fused ops regenerate their dropout masks from counters, so the recomputation rewinds the op stream
counter to the value it had in the forward pass and reproduces the same masks.

Reference: onmt/reversible_models/transformers.py:94-147 (encoder function), :267-334 (decoder function),
onmt/reversible_models/transformers.py ``ReversibleTransformerEncoderLayer`` / ``...DecoderLayer``;
tools/grad_check_reversible.py checks the same property our test checks (gradients equal those of the plain graph).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from .layers import CrossAttention, FeedForward, LayerNorm, PackedSeqs, SelfAttention


class _ReversibleFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, layer, seqs, memory, mem_seqs, n_params, *params):
        ctx.layer, ctx.seqs, ctx.mem_seqs = layer, seqs, mem_seqs
        ctx.counter = ops._Rng.counter
        ctx.has_memory = memory is not None
        with torch.no_grad():
            y1 = x1 + layer.f(x2, seqs, memory, mem_seqs)
            y2 = x2 + layer.g(y1)
        ctx.counter_end = ops._Rng.counter
        ctx.save_for_backward(y1, y2, memory if memory is not None else y1.new_zeros(0))
        return y1, y2

    @staticmethod
    def backward(ctx, dy1, dy2):
        layer, seqs = ctx.layer, ctx.seqs
        y1, y2, memory = ctx.saved_tensors
        memory = memory if ctx.has_memory else None
        saved = ops._Rng.counter
        params = [p for p in layer.parameters() if p.requires_grad]
        mem_in = memory.detach().requires_grad_(True) if memory is not None else None
        try:
            with torch.enable_grad():
                # G ran after F in the forward pass, so its dropout streams start f_streams ids after the layer's first
                ops._Rng.counter = ctx.counter + layer.f_streams
                y1_in = y1.detach().requires_grad_(True)
                g_out = layer.g(y1_in)
            x2 = (y2 - g_out).detach()
            grads_g = torch.autograd.grad(g_out, [y1_in] + params, dy2, allow_unused=True)
            dy1_total = dy1 + grads_g[0]
            with torch.enable_grad():
                ops._Rng.counter = ctx.counter
                x2_in = x2.requires_grad_(True)
                f_out = layer.f(x2_in, seqs, mem_in, ctx.mem_seqs)
            x1 = (y1 - f_out).detach()
            f_inputs = [x2_in] + params + ([mem_in] if mem_in is not None else [])
            grads_f = torch.autograd.grad(f_out, f_inputs, dy1_total, allow_unused=True)
        finally:
            ops._Rng.counter = saved
        dx1 = dy1_total
        dx2 = dy2 + grads_f[0]
        n = len(params)
        dparams = []
        for i in range(n):
            a, b = grads_g[1 + i], grads_f[1 + i]
            dparams.append(a if b is None else (b if a is None else a + b))
        dmem = grads_f[1 + n] if len(grads_f) > 1 + n else None
        layer._last_inputs = (x1, x2)      # lets the stack free its references; also used by the tests
        return (dx1, dx2, None, None, dmem, None, None) + tuple(dparams)


class ReversibleLayer(nn.Module):
    """Encoder layer (``cross=False``) or decoder layer (``cross=True``) in reversible form."""

    def __init__(self, dim, heads, inner, dropout=0.1, attn_dropout=0.1, activation="relu", causal=False, cross=False):
        super().__init__()
        self.attn_norm = LayerNorm(dim)
        self.attn = SelfAttention(dim, heads, attn_dropout, causal=causal)
        self.cross = cross
        if cross:
            self.cross_norm = LayerNorm(dim)
            self.cross_attn = CrossAttention(dim, heads, attn_dropout)
        self.ffn_norm = LayerNorm(dim)
        self.ffn = FeedForward(dim, inner, dropout, activation)
        self.dropout = dropout
        self.f_streams = 0

    def f(self, x, seqs, memory=None, mem_seqs=None):
        start = ops._Rng.counter
        h = self.attn(self.attn_norm(x), seqs, residual=None, dropout_p=self.dropout)
        if self.cross:
            h = h + self.cross_attn(self.cross_norm(x + h), seqs, memory, mem_seqs, residual=None, dropout_p=self.dropout)
        self.f_streams = ops._Rng.counter - start
        return h

    def g(self, x):
        return self.ffn(self.ffn_norm(x), residual=None, dropout_p=self.dropout)

    def forward(self, x1, x2, seqs: PackedSeqs, memory=None, mem_seqs: Optional[PackedSeqs] = None):
        if not torch.is_grad_enabled():
            y1 = x1 + self.f(x2, seqs, memory, mem_seqs)
            return y1, x2 + self.g(y1)
        params = [p for p in self.parameters() if p.requires_grad]
        return _ReversibleFn.apply(x1, x2, self, seqs, memory, mem_seqs, len(params), *params)

    def step(self, x1, x2, cache: dict, mem_mask):
        """Incremental decoding of one position (no gradients, nothing to reconstruct)."""
        h = self.attn.step(self.attn_norm(x2), cache)
        if self.cross:
            h = h + self.cross_attn.step(self.cross_norm(x2 + h), cache, mem_mask)
        y1 = x1 + h
        return y1, x2 + self.ffn(self.ffn_norm(y1), residual=None)

    def forward_plain(self, x1, x2, seqs, memory=None, mem_seqs=None):
        """The same computation through ordinary autograd (activations stored); used as the oracle in tests."""
        y1 = x1 + self.f(x2, seqs, memory, mem_seqs)
        return y1, x2 + self.g(y1)


class ReversibleStack(nn.Module):
    """``x -> (x, x)`` -> layers -> ``(y1 + y2) / 2`` -> LayerNorm."""

    def __init__(self, n_layers, dim, heads, inner, dropout=0.1, attn_dropout=0.1, activation="relu", causal=False, cross=False):
        super().__init__()
        self.layers = nn.ModuleList([ReversibleLayer(dim, heads, inner, dropout, attn_dropout, activation, causal, cross)
                                     for _ in range(n_layers)])
        self.final_norm = LayerNorm(dim)

    def forward(self, x, seqs, memory=None, mem_seqs=None, plain: bool = False):
        x1, x2 = x, x
        for layer in self.layers:
            x1, x2 = (layer.forward_plain if plain else layer)(x1, x2, seqs, memory, mem_seqs)
        return self.final_norm((x1 + x2) * 0.5)

    def step(self, x, buffers, mem_mask):
        x1, x2 = x, x
        for layer, cache in zip(self.layers, buffers):
            x1, x2 = layer.step(x1, x2, cache, mem_mask)
        return self.final_norm((x1 + x2) * 0.5)
