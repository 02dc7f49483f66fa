"""UnitY / Seamless style speech-encoder adaptor on the typed building blocks.

``UnitYTransformerAdaptorLayer`` shortens the sequence by a strided 1-D convolution followed by a GLU, once on the
residual branch and once in front of self-attention, then applies the usual pre-norm self-attention and feed-forward
sub-layers; ``UnitYEncoderAdaptor`` is an inner projection followed by a stack of such layers and a final LayerNorm.
``SeamlessSpeechEncoder`` chains a frame-level encoder (any module returning ``(states [B, T, H], padding_mask)``)
with the adaptor.

Reference: onmt/models/unity/adaptor_block.py:25-121 (``UnitYEncoderAdaptor``), :123-315 (``UnitYTransformerAdaptorLayer``),
onmt/models/unity/seamless_encoder.py, onmt/models/unity/unity_builder.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .blocks import StandardFeedForwardNetwork, StandardLayerNorm, StandardMultiheadAttention

__all__ = ["UnitYTransformerAdaptorLayer", "UnitYEncoderAdaptor", "SeamlessSpeechEncoder", "pooled_padding_mask"]


def pooled_padding_mask(padding_mask: Optional[torch.Tensor], kernel_size: int, stride: int, new_len: int):
    """Padding mask after a convolution with padding ``kernel_size // 2``: length -> floor((len + 2p - k) / stride) + 1."""
    if padding_mask is None:
        return None
    lengths = (~padding_mask).sum(1)
    pad = kernel_size // 2
    new = torch.div(lengths + 2 * pad - kernel_size, stride, rounding_mode="floor") + 1
    return torch.arange(new_len, device=padding_mask.device)[None, :] >= new.clamp(min=0)[:, None]


class UnitYTransformerAdaptorLayer(nn.Module):
    def __init__(self, model_dim: int, num_heads: int, ffn_inner_dim: int, kernel_size: int = 8, stride: int = 8, dropout_p: float = 0.1):
        super().__init__()
        self.kernel_size, self.stride = kernel_size, stride
        pad = kernel_size // 2
        self.residual_layer_norm = StandardLayerNorm(model_dim)
        self.residual_conv = nn.Conv1d(model_dim, model_dim * 2, kernel_size, stride, pad)
        self.self_attn_layer_norm = StandardLayerNorm(model_dim)
        self.self_attn_conv = nn.Conv1d(model_dim, model_dim * 2, kernel_size, stride, pad)
        self.self_attn = StandardMultiheadAttention(model_dim, num_heads, attn_dropout_p=dropout_p)
        self.ffn_layer_norm = StandardLayerNorm(model_dim)
        self.ffn = StandardFeedForwardNetwork(model_dim, ffn_inner_dim, dropout_p=dropout_p)
        self.dropout_p = dropout_p

    def _pool(self, conv, x):
        return F.glu(conv(x.transpose(1, 2)), dim=1).transpose(1, 2)

    def forward(self, x, padding_mask=None):
        residual = self._pool(self.residual_conv, self.residual_layer_norm(x))
        h = self._pool(self.self_attn_conv, self.self_attn_layer_norm(x))
        mask = pooled_padding_mask(padding_mask, self.kernel_size, self.stride, h.shape[1])
        h = self.self_attn(h, key_padding_mask=mask)
        x = residual + F.dropout(h, self.dropout_p, self.training)
        x = x + F.dropout(self.ffn(self.ffn_layer_norm(x)), self.dropout_p, self.training)
        return x, mask


class UnitYEncoderAdaptor(nn.Module):
    def __init__(self, model_dim: int, num_layers: int = 1, num_heads: int = 16, ffn_inner_dim: Optional[int] = None,
                 kernel_size: int = 8, stride: int = 8, dropout_p: float = 0.1):
        super().__init__()
        inner = ffn_inner_dim or 4 * model_dim
        self.inner_layer_norm = StandardLayerNorm(model_dim)
        self.inner_proj = nn.Linear(model_dim, inner)
        self.inner_out = nn.Linear(inner, model_dim)
        self.layers = nn.ModuleList([UnitYTransformerAdaptorLayer(model_dim, num_heads, inner, kernel_size, stride, dropout_p)
                                     for _ in range(num_layers)])
        self.layer_norm = StandardLayerNorm(model_dim)
        self.dropout_p = dropout_p

    def forward(self, x, padding_mask=None):
        h = self.inner_out(F.dropout(F.relu(self.inner_proj(self.inner_layer_norm(x))), self.dropout_p, self.training))
        x = x + 0.5 * h
        for layer in self.layers:
            x, padding_mask = layer(x, padding_mask)
        return self.layer_norm(x), padding_mask


class SeamlessSpeechEncoder(nn.Module):
    """Frame-level encoder followed by the length-reducing adaptor (what the text decoder of UnitY attends to)."""

    def __init__(self, inner: nn.Module, adaptor: UnitYEncoderAdaptor):
        super().__init__()
        self.inner, self.adaptor = inner, adaptor

    def forward(self, feats, padding_mask=None):
        x, mask = self.inner(feats, padding_mask)
        return self.adaptor(x, mask)
