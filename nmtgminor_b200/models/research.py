"""Smaller research architectures: the Universal Transformer (one shared layer applied ``layers`` times with a per-step
timing signal), the document-context ("discourse") translator with a gated fusion of the previous sentence's encoding,
and the Bayes-by-backprop output layer.

Reference: onmt/legacy/UniversalTransformer (factory :558-573), onmt/models/discourse/discourse_transformer.py +
gate_layer.py (factory :414-443), onmt/models/bayes_by_backprop/*, onmt/modules/bayes_by_backprop/{gaussian,generator}.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import DecoderLayer, Embedding, EncoderLayer, LayerNorm, PackedSeqs, sinusoidal_table
from .transformer import Generator, Seq2SeqBase, Transformer, TransformerDecoder, TransformerEncoder


class UniversalTransformer(Transformer):
    """Weights of layer 0 are reused at every depth; a sinusoidal "time" embedding of the depth index is added first."""

    def __init__(self, opt, dicts):
        super().__init__(opt, dicts)
        n_enc, n_dec = len(self.encoder.layers), len(self.decoder.layers)
        self.encoder.layers = nn.ModuleList([self.encoder.layers[0]])
        self.decoder.layers = nn.ModuleList([self.decoder.layers[0]])
        self.depth = (n_enc, n_dec)
        self.register_buffer("time_signal", sinusoidal_table(max(n_enc, n_dec), opt.model_size), persistent=False)

    def encode(self, batch):
        src = batch.packed_source()
        x = self.encoder.embed(src, self.encoder.emb_dropout)
        for t in range(self.depth[0]):
            x = self.encoder.layers[0](x + self.time_signal[t].to(x.dtype), src)
        return self.encoder.final_norm(x), src

    def forward(self, batch, **kw):
        dec = self.decoder

        def decoder_forward(tgt, memory, src):
            x = dec.embed(tgt, dec.emb_dropout)
            for t in range(self.depth[1]):
                x = dec.layers[0](x + self.time_signal[t].to(x.dtype), tgt, memory, src)
            return dec.final_norm(x)
        original = dec.forward
        dec.forward = decoder_forward
        try:
            return Seq2SeqBase.forward(self, batch, **kw)
        finally:
            dec.forward = original


class GateLayer(nn.Module):
    """g = sigmoid(W [x ; c]);  out = g * x + (1 - g) * c."""

    def __init__(self, dim):
        super().__init__()
        self.proj = nn.Linear(2 * dim, dim)
        self.norm = LayerNorm(dim)

    def forward(self, x, c):
        g = torch.sigmoid(self.proj(torch.cat([x, c], -1).float())).to(x.dtype)
        return self.norm(g * x + (1 - g) * c)


class DiscourseTransformer(Transformer):
    """Encodes the previous source sentence (``past_source``) with the same encoder, lets the current sentence attend to it
    (one cross-attention layer) and fuses the result through a gate before decoding."""

    def __init__(self, opt, dicts):
        super().__init__(opt, dicts)
        from .layers import CrossAttention
        self.past_attn_norm = LayerNorm(opt.model_size)
        self.past_attn = CrossAttention(opt.model_size, opt.n_heads, opt.attn_dropout)
        self.gate = GateLayer(opt.model_size)

    def encode(self, batch):
        src = batch.packed_source()
        ctx = self.encoder(src)
        past = batch.get("packed_past_source")
        if past is None:
            return ctx, src
        past_ctx = self.encoder(past)
        attended = self.past_attn(self.past_attn_norm(ctx), src, past_ctx, past)
        return self.gate(ctx, attended), src


class BayesianGenerator(nn.Module):
    """Output layer with a factorised Gaussian posterior over its weights; sampled by reparameterisation in training.
    ``kl()`` returns KL(q || N(0, prior_sigma^2)) for the ELBO."""

    def __init__(self, dim, vocab, prior_sigma=1.0):
        super().__init__()
        self.mu = nn.Parameter(torch.empty(vocab, dim).normal_(0, dim ** -0.5))
        self.rho = nn.Parameter(torch.full((vocab, dim), -5.0))
        self.bias = nn.Parameter(torch.zeros(vocab))
        self.prior_sigma = prior_sigma

    @property
    def weight(self):
        if self.training:
            return self.mu + F.softplus(self.rho) * torch.randn_like(self.mu)
        return self.mu

    def kl(self):
        sigma = F.softplus(self.rho)
        ps = self.prior_sigma
        return (math.log(ps) - torch.log(sigma) + (sigma ** 2 + self.mu ** 2) / (2 * ps ** 2) - 0.5).sum()

    def forward(self, hidden, log_softmax=False):
        logits = F.linear(hidden.float(), self.weight, self.bias)
        return torch.log_softmax(logits, -1) if log_softmax else logits


def register_builders(register):
    register("universal_transformer")(lambda opt, dicts: UniversalTransformer(opt, dicts))
    register("discourse_translator", "discourse_speech_transformer")(lambda opt, dicts: DiscourseTransformer(opt, dicts))
