"""Conformer encoder (``-model conformer``): FFN/2 -> self-attention -> convolution module -> FFN/2 -> LayerNorm per block,
on packed frames for the attention / FFN parts and on the padded batch for the depthwise convolution.

Reference: onmt/models/conformer/block.py (``ConformerBlock``), convolution.py (``ConformerConvolution``: pointwise
conv + GLU, depthwise conv, BatchNorm or LayerNorm, SiLU, pointwise conv), onmt/models/speech_recognizer/conformer.py:20.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import Embedding, FeedForward, LayerNorm, PackedSeqs, SelfAttention, pack_padded, sinusoidal_table
from .speech_encoders import split_audio_batch
from .transformer import TransformerDecoder


class ConformerConvolution(nn.Module):
    def __init__(self, dim: int, kernel: int = 31, norm: str = "layer_norm"):
        super().__init__()
        self.pw1 = nn.Conv1d(dim, 2 * dim, 1)
        self.dw = nn.Conv1d(dim, dim, kernel, padding=kernel // 2, groups=dim)
        self.norm = nn.BatchNorm1d(dim) if norm == "batch_norm" else nn.GroupNorm(1, dim)
        self.pw2 = nn.Conv1d(dim, dim, 1)

    def forward(self, x_bt, valid):            # [B, T, C], valid [B, T]
        x = x_bt.float() * valid.unsqueeze(-1)
        x = F.glu(self.pw1(x.transpose(1, 2)), dim=1)
        x = self.dw(x * valid.unsqueeze(1))
        x = F.silu(self.norm(x))
        return self.pw2(x).transpose(1, 2)


class ConformerBlock(nn.Module):
    def __init__(self, dim, heads, inner, dropout=0.1, attn_dropout=0.1, kernel=31):
        super().__init__()
        self.ffn1_norm, self.ffn1 = LayerNorm(dim), FeedForward(dim, inner, dropout, "silu")
        self.attn_norm, self.attn = LayerNorm(dim), SelfAttention(dim, heads, attn_dropout, bias=True)
        self.conv_norm, self.conv = LayerNorm(dim), ConformerConvolution(dim, kernel)
        self.ffn2_norm, self.ffn2 = LayerNorm(dim), FeedForward(dim, inner, dropout, "silu")
        self.final_norm = LayerNorm(dim)
        self.dropout = dropout

    def forward(self, x, seqs: PackedSeqs):
        from ..ops.reference import unpad_packed
        x = x + 0.5 * (self.ffn1(self.ffn1_norm(x), dropout_p=self.dropout))
        x = self.attn(self.attn_norm(x), seqs, residual=x, dropout_p=self.dropout)
        padded = seqs.pad(self.conv_norm(x), time_first=False)
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
        valid = (torch.arange(padded.shape[1], device=x.device)[None, :] < lengths[:, None]).float()
        c = unpad_packed(self.conv(padded, valid).to(x.dtype), seqs.cu, x.shape[0])
        x = x + F.dropout(c, self.dropout, self.training)
        x = x + 0.5 * (self.ffn2(self.ffn2_norm(x), dropout_p=self.dropout))
        return self.final_norm(x)


class ConformerEncoder(nn.Module):
    def __init__(self, opt, input_size: int):
        super().__init__()
        dim = opt.model_size
        self.sub = nn.Sequential(nn.Conv2d(1, 32, 3, stride=2, padding=1), nn.ReLU(), nn.Conv2d(32, 32, 3, stride=2, padding=1), nn.ReLU())
        self.proj = nn.Linear(((input_size + 1) // 2 + 1) // 2 * 32, dim)
        n = opt.encoder_layers if getattr(opt, "encoder_layers", -1) > 0 else opt.layers
        self.register_buffer("positions", sinusoidal_table(4096, dim), persistent=False)
        self.layers = nn.ModuleList([ConformerBlock(dim, opt.n_heads, opt.inner_size, opt.dropout, opt.attn_dropout,
                                                    getattr(opt, "conv_kernel", 31)) for _ in range(n)])
        self.dim = dim

    def forward(self, source):
        feats, lengths = split_audio_batch(source)
        x = self.sub(feats.unsqueeze(1).float())
        x = x.permute(0, 2, 1, 3).reshape(x.shape[0], x.shape[2], -1)
        lengths = torch.div(torch.div(lengths + 1, 2, rounding_mode="floor") + 1, 2, rounding_mode="floor").clamp(max=x.shape[1])
        x = self.proj(x)
        x = x + self.positions[:x.shape[1]].to(x.dtype)
        packed, seqs = pack_padded(x, lengths)
        if packed.is_cuda and ops.fused_param(self.layers[0].final_norm.weight):
            packed = packed.to(torch.bfloat16)
        for layer in self.layers:
            packed = layer(packed, seqs)
        return packed, seqs


def register_builders(register):
    @register("conformer")
    def _conformer(opt, dicts):
        from .pretrained import SpeechToTextModel
        enc = ConformerEncoder(opt, getattr(opt, "input_size", 40))
        dec = TransformerDecoder(opt, Embedding(dicts["tgt"].size(), opt.model_size, getattr(opt, "pad_idx", 0)))
        return SpeechToTextModel(opt, enc, dec, dicts["tgt"].size())
