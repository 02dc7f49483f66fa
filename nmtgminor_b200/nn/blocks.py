"""Typed Transformer building blocks on padded ``[B, T, H]`` tensors: embeddings, projections, position encoders
(sinusoidal, learned, rotary), attention-mask factories (causal, ALiBi), multi-head attention with grouped key/value
heads and incremental state, dense and gated feed-forward networks, norm-order aware encoder / decoder stacks.

These are the pieces the NLLB, LLaMA and UnitY-style builders assemble.  Linear layers run the tcgen05 GEMM when their
parameters carry bf16 working copies (``nmtgminor_b200.parallel.flat.FlatParameterStore``); attention with rotary
positions or additive masks uses PyTorch's scaled-dot-product attention.

Reference: onmt/nn/embedding.py:23-143, projection.py:16-160, normalization.py:20-163, position_encoder.py:24-560,
onmt/nn/transformer/attention_mask.py:15-392, multihead_attention.py:33-614, ffn.py:20-212, norm_order.py:10,
encoder.py:90-422, decoder.py:38-509, frontend.py:19-134, model.py:26-111, decoder_model.py:24-103.
"""
from __future__ import annotations

import math
from enum import Enum
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .attention import (SDPA, AttentionWeightStoreHook, ModuleList, NaiveSDPA, RelativePositionalEncoding, RelativePositionSDPA,
                        ShawRelativePositionSDPA, TorchSDPA, create_default_sdpa, default_sdpa_factory, set_default_sdpa_factory)

__all__ = ["TransformerNormOrder", "StandardEmbedding", "Linear", "TiedProjection", "StandardLayerNorm", "RMSNorm",
           "SinusoidalPositionEncoder", "LearnedPositionEncoder", "RotaryEncoder", "CausalAttentionMaskFactory",
           "ALiBiMaskFactory", "StandardMultiheadAttention", "StandardFeedForwardNetwork", "GLUFeedForwardNetwork",
           "TransformerEmbeddingFrontend", "StandardTransformerEncoderLayer", "StandardTransformerEncoder",
           "StandardTransformerDecoderLayer", "StandardTransformerDecoder", "TransformerModel", "TransformerDecoderModel",
           "IncrementalState", "padding_mask_from_lengths", "SDPA", "TorchSDPA", "NaiveSDPA", "RelativePositionSDPA",
           "RelativePositionalEncoding", "ShawRelativePositionSDPA", "AttentionWeightStoreHook", "ModuleList",
           "set_default_sdpa_factory", "create_default_sdpa", "default_sdpa_factory"]


class TransformerNormOrder(Enum):
    POST = 0
    PRE = 1
    PRE_WITH_NORMFORMER = 2


IncrementalState = Dict[int, Dict[str, torch.Tensor]]


def padding_mask_from_lengths(lengths: torch.Tensor, max_len: Optional[int] = None) -> torch.Tensor:
    """True at padded positions, ``[B, T]``."""
    T = int(max_len if max_len is not None else lengths.max())
    return torch.arange(T, device=lengths.device)[None, :] >= lengths[:, None]


class StandardEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, pad_idx: Optional[int] = None, scaled: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))
        self.pad_idx = pad_idx
        nn.init.normal_(self.weight, std=embedding_dim ** -0.5 if scaled else 1.0)
        if pad_idx is not None:
            with torch.no_grad():
                self.weight[pad_idx].zero_()

    def forward(self, x):
        return F.embedding(x, self.weight, self.pad_idx)


class Linear(nn.Module):
    """Projection over the last axis of any-rank input; fused GEMM path for parameters with bf16 working copies."""

    def __init__(self, input_dim: int, output_dim: int, bias: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(output_dim, input_dim))
        self.bias = nn.Parameter(torch.zeros(output_dim)) if bias else None
        nn.init.xavier_uniform_(self.weight)

    def forward(self, x):
        if ops.fused_param(self.weight) and x.is_cuda:
            y = ops.linear(x.reshape(-1, x.shape[-1]), self.weight, self.bias)
            return y.view(*x.shape[:-1], -1)
        return F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


class TiedProjection(nn.Module):
    def __init__(self, weight: nn.Parameter, bias: Optional[nn.Parameter] = None):
        super().__init__()
        self.weight, self.bias = weight, bias

    def forward(self, x):
        return F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


class StandardLayerNorm(nn.LayerNorm):
    pass


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, bias: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim)) if bias else None
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        y = y.to(x.dtype) * self.weight.to(x.dtype)
        return y if self.bias is None else y + self.bias.to(x.dtype)


# ---- position encoders ------------------------------------------------------------------------------------
class SinusoidalPositionEncoder(nn.Module):
    """fairseq-style table (sin half, cos half); positions start at ``1 + pad offset`` as in fairseq when legacy."""

    def __init__(self, dim: int, max_seq_len: int, legacy_pad_idx: Optional[int] = None):
        super().__init__()
        start = 1 + legacy_pad_idx if legacy_pad_idx is not None else 0
        half = dim // 2
        freq = torch.exp(torch.arange(half, dtype=torch.float32) * -(math.log(10000.0) / max(half - 1, 1)))
        pos = torch.arange(start, start + max_seq_len, dtype=torch.float32)[:, None] * freq[None, :]
        table = torch.cat([pos.sin(), pos.cos()], -1)
        if dim % 2:
            table = F.pad(table, (0, 1))
        self.register_buffer("table", table, persistent=False)

    def forward(self, x, state_offset: int = 0):
        return x + self.table[state_offset:state_offset + x.shape[1]].to(x.dtype)[None]


class LearnedPositionEncoder(nn.Module):
    def __init__(self, dim: int, max_seq_len: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(max_seq_len, dim))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x, state_offset: int = 0):
        return x + self.weight[state_offset:state_offset + x.shape[1]].to(x.dtype)[None]


class RotaryEncoder(nn.Module):
    """Rotates consecutive feature pairs of ``[B, heads, T, d]`` by position-dependent angles."""

    def __init__(self, dim: int, max_seq_len: int, theta: float = 10000.0):
        super().__init__()
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        ang = torch.arange(max_seq_len, dtype=torch.float32)[:, None] * inv[None, :]
        self.register_buffer("cos", ang.cos(), persistent=False)
        self.register_buffer("sin", ang.sin(), persistent=False)

    def forward(self, x, state_offset: int = 0):
        T = x.shape[-2]
        cos = self.cos[state_offset:state_offset + T].to(x.dtype)
        sin = self.sin[state_offset:state_offset + T].to(x.dtype)
        x1, x2 = x[..., 0::2], x[..., 1::2]
        out = torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1)
        return out.flatten(-2)


# ---- attention masks --------------------------------------------------------------------------------------
class CausalAttentionMaskFactory:
    def __call__(self, q_len: int, k_len: int, device, dtype=torch.float32) -> torch.Tensor:
        """Additive ``[q_len, k_len]`` mask; query i (the last q_len positions of the keys) sees keys <= its position."""
        i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
        j = torch.arange(k_len, device=device)[None, :]
        return torch.zeros(q_len, k_len, device=device, dtype=dtype).masked_fill(j > i, float("-inf"))


class ALiBiMaskFactory:
    """Causal mask plus per-head linear distance penalties (slopes 2^(-8 h / H))."""

    def __init__(self, num_heads: int):
        self.num_heads = num_heads

    @staticmethod
    def slopes(n: int) -> torch.Tensor:
        def pow2(k):
            start = 2.0 ** (-(2.0 ** -(math.log2(k) - 3)))
            return [start * (start ** i) for i in range(k)]
        if math.log2(n).is_integer():
            return torch.tensor(pow2(n))
        k = 2 ** math.floor(math.log2(n))
        return torch.tensor(pow2(k) + pow2(2 * k)[0::2][:n - k])

    def __call__(self, q_len: int, k_len: int, device, dtype=torch.float32) -> torch.Tensor:
        causal = CausalAttentionMaskFactory()(q_len, k_len, device, dtype)
        i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
        j = torch.arange(k_len, device=device)[None, :]
        dist = (j - i).clamp(max=0).to(dtype)                                   # <= 0 for visible keys
        return causal[None] + self.slopes(self.num_heads).to(device=device, dtype=dtype)[:, None, None] * dist[None]


# ---- attention --------------------------------------------------------------------------------------------
class StandardMultiheadAttention(nn.Module):
    """Multi-head attention with optional grouped key/value heads, rotary position encoder and incremental state.

    ``forward(x, keys, values, key_padding_mask, attn_mask, state)``; with ``state`` (a dict) the projected keys /
    values are appended to ``state['k'] / state['v']`` (self-attention) or computed once (``static_kv``)."""

    def __init__(self, model_dim: int, num_heads: int, num_key_value_heads: Optional[int] = None, pos_encoder=None,
                 bias: bool = True, attn_dropout_p: float = 0.0, static_kv: bool = False, sdpa=None):
        super().__init__()
        from .attention import create_default_sdpa
        self.sdpa = sdpa if sdpa is not None else create_default_sdpa(attn_dropout_p=attn_dropout_p)
        self._attn_weight_hooks = {}
        self.num_heads = num_heads
        self.num_kv_heads = num_key_value_heads or num_heads
        assert num_heads % self.num_kv_heads == 0 and model_dim % num_heads == 0
        self.head_dim = model_dim // num_heads
        self.q_proj = Linear(model_dim, model_dim, bias)
        self.k_proj = Linear(model_dim, self.head_dim * self.num_kv_heads, bias)
        self.v_proj = Linear(model_dim, self.head_dim * self.num_kv_heads, bias)
        self.output_proj = Linear(model_dim, model_dim, bias)
        self.pos_encoder = pos_encoder
        self.attn_dropout_p = attn_dropout_p
        self.static_kv = static_kv

    def _split(self, x, heads):
        B, T, _ = x.shape
        return x.view(B, T, heads, self.head_dim).transpose(1, 2)

    def register_attn_weight_hook(self, hook):
        """``hook(module, attn, attn_weights)`` runs after every forward pass; returns a handle with ``remove()``.  With a
        hook registered the attention weights are materialised (the fused PyTorch attention does not return them)."""
        key = id(hook)
        self._attn_weight_hooks[key] = hook
        owner = self

        class _Handle:
            def remove(self_inner):
                owner._attn_weight_hooks.pop(key, None)
        return _Handle()

    def forward(self, x, keys=None, values=None, key_padding_mask=None, attn_mask=None, state: Optional[dict] = None):
        keys = x if keys is None else keys
        values = keys if values is None else values
        offset = 0
        q = self._split(self.q_proj(x), self.num_heads)
        if state is not None and self.static_kv and "k" in state:
            k, v = state["k"], state["v"]
        else:
            k = self._split(self.k_proj(keys), self.num_kv_heads)
            v = self._split(self.v_proj(values), self.num_kv_heads)
            if state is not None and not self.static_kv and "k" in state:
                offset = state["k"].shape[2]
            if self.pos_encoder is not None:
                k = self.pos_encoder(k, offset)
            if state is not None:
                if not self.static_kv and "k" in state:
                    k, v = torch.cat([state["k"], k], 2), torch.cat([state["v"], v], 2)
                state["k"], state["v"] = k, v
        if self.pos_encoder is not None:
            q = self.pos_encoder(q, offset)
        if self.num_kv_heads != self.num_heads:
            rep = self.num_heads // self.num_kv_heads
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        mask = None
        if attn_mask is not None:
            mask = attn_mask.to(q.dtype)
            mask = mask[None, None] if mask.dim() == 2 else mask[None]
        if key_padding_mask is not None:
            pad = torch.zeros(key_padding_mask.shape, dtype=q.dtype, device=q.device).masked_fill(key_padding_mask, float("-inf"))
            mask = pad[:, None, None, :] if mask is None else mask + pad[:, None, None, :]
        out, weights = self.sdpa(q, k, v, mask, needs_weights=bool(self._attn_weight_hooks))
        for hook in list(self._attn_weight_hooks.values()):
            hook(self, out, weights)
        return self.output_proj(out.transpose(1, 2).reshape(x.shape[0], x.shape[1], -1))


# ---- feed-forward -----------------------------------------------------------------------------------------
class StandardFeedForwardNetwork(nn.Module):
    def __init__(self, model_dim: int, inner_dim: int, bias: bool = True, activation: str = "relu", dropout_p: float = 0.0,
                 norm_order: TransformerNormOrder = TransformerNormOrder.PRE):
        super().__init__()
        self.inner_proj, self.output_proj = Linear(model_dim, inner_dim, bias), Linear(inner_dim, model_dim, bias)
        self.activation, self.dropout_p = activation, dropout_p
        self.inner_norm = StandardLayerNorm(inner_dim) if norm_order == TransformerNormOrder.PRE_WITH_NORMFORMER else None

    def forward(self, x):
        w1, w2 = self.inner_proj, self.output_proj
        if (self.inner_norm is None and ops.fused_param(w1.weight) and x.is_cuda and self.activation in ("relu", "gelu", "silu")):
            y = ops.mlp(x.reshape(-1, x.shape[-1]), w1.weight, w1.bias, w2.weight, w2.bias, self.activation, self.dropout_p, 0.0,
                        None, self.training)
            return y.view_as(x)
        h = getattr(F, self.activation)(w1(x))
        if self.inner_norm is not None:
            h = self.inner_norm(h)
        return w2(F.dropout(h, self.dropout_p, self.training))


class GLUFeedForwardNetwork(nn.Module):
    """``output(act(gate(x)) * inner(x))``; the inner dimension is optionally scaled and rounded up (LLaMA)."""

    def __init__(self, model_dim: int, inner_dim: int, bias: bool = False, activation: str = "silu", inner_dim_scale: float = 2 / 3,
                 inner_dim_to_multiple: int = 1, dropout_p: float = 0.0):
        super().__init__()
        inner = int(inner_dim * inner_dim_scale)
        if inner_dim_to_multiple > 1:
            inner = inner_dim_to_multiple * ((inner + inner_dim_to_multiple - 1) // inner_dim_to_multiple)
        self.inner_dim = inner
        self.gate_proj, self.inner_proj = Linear(model_dim, inner, bias), Linear(model_dim, inner, bias)
        self.output_proj = Linear(inner, model_dim, bias)
        self.activation, self.dropout_p = activation, dropout_p

    def forward(self, x):
        h = getattr(F, self.activation)(self.gate_proj(x)) * self.inner_proj(x)
        return self.output_proj(F.dropout(h, self.dropout_p, self.training))


# ---- front end and stacks ---------------------------------------------------------------------------------
class TransformerEmbeddingFrontend(nn.Module):
    def __init__(self, embed: StandardEmbedding, pos_encoder=None, no_scale: bool = False, layer_norm: bool = False,
                 dropout_p: float = 0.1):
        super().__init__()
        self.embed, self.pos_encoder = embed, pos_encoder
        self.scale = 1.0 if no_scale else math.sqrt(embed.weight.shape[1])
        self.layer_norm = StandardLayerNorm(embed.weight.shape[1]) if layer_norm else None
        self.dropout_p = dropout_p

    def forward(self, tokens, lengths=None, state_offset: int = 0):
        x = self.embed(tokens) * self.scale
        if self.pos_encoder is not None:
            x = self.pos_encoder(x, state_offset)
        if self.layer_norm is not None:
            x = self.layer_norm(x)
        x = F.dropout(x, self.dropout_p, self.training)
        mask = padding_mask_from_lengths(lengths, tokens.shape[1]) if lengths is not None else None
        return x, mask


def _norm(factory, dim):
    return factory(dim) if factory is not None else StandardLayerNorm(dim)


class StandardTransformerEncoderLayer(nn.Module):
    def __init__(self, self_attn, ffn, model_dim: int, dropout_p: float = 0.1,
                 norm_order: TransformerNormOrder = TransformerNormOrder.POST, layer_norm_factory=None):
        super().__init__()
        self.self_attn, self.ffn, self.norm_order, self.dropout_p = self_attn, ffn, norm_order, dropout_p
        self.self_attn_layer_norm = _norm(layer_norm_factory, model_dim)
        self.ffn_layer_norm = _norm(layer_norm_factory, model_dim)
        self.self_attn_norm = _norm(layer_norm_factory, model_dim) if norm_order == TransformerNormOrder.PRE_WITH_NORMFORMER else None

    def forward(self, x, padding_mask=None, attn_mask=None):
        post = self.norm_order == TransformerNormOrder.POST
        r = x
        h = x if post else self.self_attn_layer_norm(x)
        h = self.self_attn(h, key_padding_mask=padding_mask, attn_mask=attn_mask)
        if self.self_attn_norm is not None:
            h = self.self_attn_norm(h)
        x = r + F.dropout(h, self.dropout_p, self.training)
        if post:
            x = self.self_attn_layer_norm(x)
        r = x
        h = self.ffn(x if post else self.ffn_layer_norm(x))
        x = r + F.dropout(h, self.dropout_p, self.training)
        return self.ffn_layer_norm(x) if post else x


class StandardTransformerEncoder(nn.Module):
    def __init__(self, layers, model_dim: int, norm_order: TransformerNormOrder = TransformerNormOrder.POST,
                 layer_norm_factory=None, layer_drop_p: float = 0.0):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.layer_norm = _norm(layer_norm_factory, model_dim) if norm_order != TransformerNormOrder.POST else None
        self.layer_drop_p = layer_drop_p

    def forward(self, x, padding_mask=None):
        for layer in self.layers:
            if self.training and self.layer_drop_p > 0 and torch.rand(()) < self.layer_drop_p:
                continue
            x = layer(x, padding_mask)
        return (self.layer_norm(x) if self.layer_norm is not None else x), padding_mask


class StandardTransformerDecoderLayer(nn.Module):
    def __init__(self, self_attn, encoder_decoder_attn, ffn, model_dim: int, dropout_p: float = 0.1,
                 norm_order: TransformerNormOrder = TransformerNormOrder.POST, layer_norm_factory=None):
        super().__init__()
        self.self_attn, self.encoder_decoder_attn, self.ffn = self_attn, encoder_decoder_attn, ffn
        self.norm_order, self.dropout_p = norm_order, dropout_p
        self.self_attn_layer_norm = _norm(layer_norm_factory, model_dim)
        self.encoder_decoder_attn_layer_norm = _norm(layer_norm_factory, model_dim) if encoder_decoder_attn is not None else None
        self.ffn_layer_norm = _norm(layer_norm_factory, model_dim)

    def forward(self, x, padding_mask=None, self_attn_mask=None, encoder_output=None, encoder_padding_mask=None,
                state: Optional[dict] = None):
        post = self.norm_order == TransformerNormOrder.POST
        drop = lambda t: F.dropout(t, self.dropout_p, self.training)
        sa_state = None if state is None else state.setdefault("self", {})
        r = x
        h = self.self_attn(x if post else self.self_attn_layer_norm(x), key_padding_mask=padding_mask, attn_mask=self_attn_mask,
                           state=sa_state)
        x = r + drop(h)
        if post:
            x = self.self_attn_layer_norm(x)
        if self.encoder_decoder_attn is not None:
            ca_state = None if state is None else state.setdefault("cross", {})
            r = x
            h = self.encoder_decoder_attn(x if post else self.encoder_decoder_attn_layer_norm(x), encoder_output, encoder_output,
                                          key_padding_mask=encoder_padding_mask, state=ca_state)
            x = r + drop(h)
            if post:
                x = self.encoder_decoder_attn_layer_norm(x)
        r = x
        x = r + drop(self.ffn(x if post else self.ffn_layer_norm(x)))
        return self.ffn_layer_norm(x) if post else x


class StandardTransformerDecoder(nn.Module):
    def __init__(self, layers, model_dim: int, norm_order: TransformerNormOrder = TransformerNormOrder.POST,
                 layer_norm_factory=None, self_attn_mask_factory=None):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.layer_norm = _norm(layer_norm_factory, model_dim) if norm_order != TransformerNormOrder.POST else None
        self.self_attn_mask_factory = self_attn_mask_factory or CausalAttentionMaskFactory()

    def forward(self, x, padding_mask=None, encoder_output=None, encoder_padding_mask=None, state: Optional[IncrementalState] = None):
        past = 0
        if state is not None and 0 in state and "k" in state[0].get("self", {}):
            past = state[0]["self"]["k"].shape[2]
        mask = self.self_attn_mask_factory(x.shape[1], past + x.shape[1], x.device, torch.float32)
        for i, layer in enumerate(self.layers):
            st = None if state is None else state.setdefault(i, {})
            x = layer(x, padding_mask if state is None else None, mask, encoder_output, encoder_padding_mask, st)
        return (self.layer_norm(x) if self.layer_norm is not None else x), padding_mask


class TransformerModel(nn.Module):
    """Encoder-decoder model assembled from front ends, stacks and a final projection."""

    def __init__(self, encoder_frontend, encoder, decoder_frontend, decoder, final_proj, target_pad_idx: Optional[int] = 0):
        super().__init__()
        self.encoder_frontend, self.encoder = encoder_frontend, encoder
        self.decoder_frontend, self.decoder, self.final_proj = decoder_frontend, decoder, final_proj
        self.target_pad_idx = target_pad_idx

    def encode(self, src_tokens, src_lengths=None):
        x, mask = self.encoder_frontend(src_tokens, src_lengths)
        return self.encoder(x, mask)

    def decode(self, tgt_tokens, encoder_output, encoder_padding_mask, tgt_lengths=None, state: Optional[IncrementalState] = None):
        offset = 0
        if state is not None and 0 in state and "k" in state[0].get("self", {}):
            offset = state[0]["self"]["k"].shape[2]
        x, mask = self.decoder_frontend(tgt_tokens, tgt_lengths, state_offset=offset)
        x, _ = self.decoder(x, mask, encoder_output, encoder_padding_mask, state)
        return self.final_proj(x)

    def forward(self, src_tokens, src_lengths, tgt_tokens, tgt_lengths=None):
        enc, enc_mask = self.encode(src_tokens, src_lengths)
        return self.decode(tgt_tokens, enc, enc_mask, tgt_lengths)

    @torch.no_grad()
    def greedy(self, src_tokens, src_lengths, bos: int, eos: int, max_len: int = 64):
        enc, enc_mask = self.encode(src_tokens, src_lengths)
        B = src_tokens.shape[0]
        out = torch.full((B, 1), bos, dtype=torch.long, device=src_tokens.device)
        state: IncrementalState = {}
        done = torch.zeros(B, dtype=torch.bool, device=src_tokens.device)
        for _ in range(max_len):
            logits = self.decode(out[:, -1:], enc, enc_mask, state=state)
            nxt = logits[:, -1].argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, eos), nxt)
            out = torch.cat([out, nxt[:, None]], 1)
            done |= nxt == eos
            if bool(done.all()):
                break
        return out


class TransformerDecoderModel(nn.Module):
    """Decoder-only language model (LLaMA family)."""

    def __init__(self, decoder_frontend, decoder, final_proj, target_pad_idx: Optional[int] = None):
        super().__init__()
        self.decoder_frontend, self.decoder, self.final_proj = decoder_frontend, decoder, final_proj
        self.target_pad_idx = target_pad_idx

    def forward(self, tokens, lengths=None, state: Optional[IncrementalState] = None):
        offset = 0
        if state is not None and 0 in state and "k" in state[0].get("self", {}):
            offset = state[0]["self"]["k"].shape[2]
        x, mask = self.decoder_frontend(tokens, lengths, state_offset=offset)
        x, _ = self.decoder(x, mask, state=state)
        return self.final_proj(x)

    @torch.no_grad()
    def generate(self, prompt, max_new_tokens: int = 32, eos: Optional[int] = None):
        state: IncrementalState = {}
        out = prompt
        logits = self.forward(prompt, state=state)
        for _ in range(max_new_tokens):
            nxt = logits[:, -1].argmax(-1, keepdim=True)
            out = torch.cat([out, nxt], 1)
            if eos is not None and bool((nxt == eos).all()):
                break
            logits = self.forward(nxt, state=state)
        return out
