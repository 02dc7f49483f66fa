"""Speech encoders on packed frames: wav2vec 2.0 family (wav2vec2 / HuBERT / WavLM-style), Whisper, and the
plain speech Transformer front-ends (linear projection of stacked filterbanks or 2 x Conv2d subsampling).

All encoders take the batch's ``source`` tensor ``[T, B, 1 + F]`` (channel 0 = 1 for real frames / samples, 0 for
padding; the rest are features or the raw waveform), run their convolutional front-end on the padded batch
(cuDNN through PyTorch), then drop the padding once and run every Transformer layer on packed
``[frames, hidden]`` matrices with the variable-length attention kernel - the "unpad once" execution that the
reference only reaches when its fp16 flash path is available
(onmt/models/speech_recognizer/fairseq_wav2vec2/wav2vec2.py:998-1034).

Reference behaviour: wav2vec2 ``Wav2Vec2Model`` / ``ConvFeatureExtractionModel`` / ``TransformerEncoder``
(fairseq_wav2vec2/wav2vec2.py:91-731, :733-811, :814-1142), wrapper ``FairseqWav2Vec``
(onmt/models/speech_recognizer/wav2vec2.py:165-519), HuBERT / WavLM wrappers (hubert.py:93, wavlm.py:56);
``WhisperEncoder`` (onmt/models/whisper/whisper_encoder.py:545-744); speech Transformer front-ends
(onmt/models/transformers.py:90-147).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import EncoderLayer, LayerNorm, Linear, PackedSeqs, SelfAttention, pack_padded, sinusoidal_table

W2V_LARGE_CONV = [(512, 10, 5)] + [(512, 3, 2)] * 4 + [(512, 2, 2)] * 2


def split_audio_batch(source):
    """``[T, B, 1 + F]`` -> features ``[B, T, F]``, lengths ``[B]``."""
    mask = source[:, :, 0] > 0
    lengths = mask.sum(0).to(torch.int64)
    return source[:, :, 1:].transpose(0, 1).contiguous(), lengths


def compute_mask_spans(B: int, T: int, lengths, mask_prob: float, mask_length: int, generator=None):
    """SpecAugment-style time masks: for each utterance ~mask_prob * len / mask_length spans of mask_length frames."""
    mask = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        L = int(lengths[b])
        n = int(mask_prob * L / max(mask_length, 1) + torch.rand(1, generator=generator).item())
        if n <= 0 or L <= mask_length:
            continue
        starts = torch.randint(0, L - mask_length + 1, (n,), generator=generator)
        for s in starts.tolist():
            mask[b, s:s + mask_length] = True
    return mask


class ConvFeatureExtractor(nn.Module):
    """7-layer strided Conv1d stack over the raw waveform (total stride 320).  ``mode='layer_norm'`` normalises every
    layer's channels; ``mode='default'`` applies GroupNorm on the first layer only."""

    def __init__(self, conv_layers=W2V_LARGE_CONV, mode: str = "layer_norm", conv_bias: bool = False):
        super().__init__()
        self.specs = list(conv_layers)
        self.mode = mode
        self.convs = nn.ModuleList()
        self.norms = nn.ModuleList()
        c_in = 1
        for i, (c, k, s) in enumerate(self.specs):
            conv = nn.Conv1d(c_in, c, k, stride=s, bias=conv_bias)
            nn.init.kaiming_normal_(conv.weight)
            self.convs.append(conv)
            if mode == "layer_norm":
                self.norms.append(nn.LayerNorm(c))
            elif i == 0:
                self.norms.append(nn.GroupNorm(c, c))
            else:
                self.norms.append(nn.Identity())
            c_in = c
        self.out_dim = c_in

    def output_lengths(self, lengths):
        for _, k, s in self.specs:
            lengths = torch.div(lengths - k, s, rounding_mode="floor") + 1
        return lengths.clamp(min=0)

    def forward(self, wav):          # [B, samples] -> [B, T', C]
        if wav.is_cuda and len(self.convs) > 1 and ops.fused_param(self.convs[1].weight):
            return self._forward_gemm(wav)
        x = wav.unsqueeze(1)
        for conv, norm in zip(self.convs, self.norms):
            x = conv(x)
            if isinstance(norm, nn.LayerNorm):
                x = norm(x.transpose(1, 2)).transpose(1, 2)
            else:
                x = norm(x)
            x = F.gelu(x)
        return x.transpose(1, 2)


    def _forward_gemm(self, wav):
        """Channels-last path: the single-channel first layer stays a library convolution, every later layer is one
        tcgen05 GEMM over overlapping rows (``ops.conv.conv1d``) with GELU in its epilogue when no norm intervenes."""
        from ..ops.conv import conv1d
        conv, norm = self.convs[0], self.norms[0]
        x = F.conv1d(wav.unsqueeze(1).to(conv.weight.dtype), conv.weight, conv.bias, stride=conv.stride[0])
        if isinstance(norm, nn.LayerNorm):
            x = F.gelu(norm(x.transpose(1, 2)))
        else:
            x = F.gelu(norm(x)).transpose(1, 2)
        x = x.to(torch.bfloat16)
        for conv, norm in zip(self.convs[1:], self.norms[1:]):
            if isinstance(norm, nn.LayerNorm):
                x = conv1d(x, conv.weight, conv.bias, conv.stride[0], "none")
                x = F.gelu(F.layer_norm(x.float(), norm.normalized_shape, norm.weight.float(), norm.bias.float(), norm.eps)).to(torch.bfloat16)
            else:
                x = conv1d(x, conv.weight, conv.bias, conv.stride[0], "gelu")
        return x.float()      # the modules that follow (feature LayerNorm, projection) hold fp32 parameters


class ConvPositionalEmbedding(nn.Module):
    """Grouped Conv1d (k = 128, 16 groups) with weight normalisation + GELU, added to the frame embeddings."""

    def __init__(self, dim: int, kernel: int = 128, groups: int = 16):
        super().__init__()
        conv = nn.Conv1d(dim, dim, kernel, padding=kernel // 2, groups=groups)
        nn.init.normal_(conv.weight, 0, math.sqrt(4.0 / (kernel * dim)))
        nn.init.zeros_(conv.bias)
        self.conv = nn.utils.parametrizations.weight_norm(conv, name="weight", dim=2)
        self.trim = 1 if kernel % 2 == 0 else 0

    def forward(self, x_bt):          # [B, T, C]
        y = self.conv(x_bt.transpose(1, 2))
        if self.trim:
            y = y[:, :, :-self.trim]
        return F.gelu(y).transpose(1, 2)


class GatedRelPosSelfAttention(SelfAttention):
    """WavLM self-attention: a bucketed relative-position bias (one ``[buckets, heads]`` table owned by the first
    layer and shared by all) is added to the scores after being scaled, per query position and head, by a gate
    computed from the query: ``g = a * (b * grep_a - 1) + 2`` with ``a, b = sigmoid(sum_4(W q))``.

    The bias goes into the attention kernels as an additive fp32 operand ``[batch, heads, T, T]`` (``ops.self_attention(...,
    bias=)``: added to the scaled scores in the softmax, its gradient returned in the same layout), so this sub-layer stays
    on the packed tensor-core path; on the CPU the PyTorch restatement takes the same argument.
    Reference: onmt/models/speech_recognizer/fairseq_wav2vec2/wavlm_modules.py:128-166 (buckets, bias), :236-256 (gate).
    """

    def __init__(self, dim, heads, attn_dropout=0.0, num_buckets=320, max_distance=800, table_owner=None):
        super().__init__(dim, heads, attn_dropout, bias=True)
        self.num_buckets, self.max_distance = num_buckets, max_distance
        self.relative_attention_bias = nn.Embedding(num_buckets, heads) if table_owner is None else None
        self._owner = [self if table_owner is None else table_owner]       # in a list: not a registered sub-module
        self.grep_linear = nn.Linear(dim // heads, 8)
        self.grep_a = nn.Parameter(torch.ones(1, heads, 1, 1))
        self._bias_cache = None

    def _buckets(self, rel):
        nb = self.num_buckets // 2
        out = (rel > 0).long() * nb
        rel = rel.abs()
        max_exact = nb // 2
        large = max_exact + (torch.log(rel.float().clamp(min=1) / max_exact) / math.log(self.max_distance / max_exact)
                             * (nb - max_exact)).long()
        large = large.clamp(max=nb - 1)
        return out + torch.where(rel < max_exact, rel, large)

    def position_bias(self, T: int, device, key):
        owner = self._owner[0]
        if owner._bias_cache is not None and owner._bias_cache[0] == key:
            return owner._bias_cache[1]
        pos = torch.arange(T, device=device)
        bias = owner.relative_attention_bias(owner._buckets(pos[None, :] - pos[:, None])).permute(2, 0, 1)    # [heads, T, T]
        owner._bias_cache = (key, bias)
        return bias

    def forward(self, x, seqs: PackedSeqs, residual=None, dropout_p: float = 0.0):
        from ..ops.reference import pad_packed
        H, h = self.dim, self.heads
        qkv = self.qkv(x)                                                          # packed [N, 3H]
        T = int(seqs.max_len)
        # the gate is a function of the query row; only the [B, h, T, T] bias itself needs the padded layout
        q_rows = qkv[:, :H].float().view(-1, h, H // h)
        gate = self.grep_linear(q_rows).view(-1, h, 2, 4).sum(-1)
        ga, gb = torch.sigmoid(gate).chunk(2, dim=-1)                              # [N, h, 1]
        scale_rows = (ga * (gb * self.grep_a.view(1, h, 1) - 1.0) + 2.0).squeeze(-1)   # [N, h]
        scale_pad, _ = pad_packed(scale_rows, seqs.cu, T)                          # [B, T, h]
        table = self.position_bias(T, x.device, (id(seqs), torch.is_grad_enabled())).float()    # [h, T, T]
        bias = scale_pad.permute(0, 2, 1).unsqueeze(-1) * table[None]               # [B, h, T, T]
        ctx = ops.self_attention(qkv, seqs.cu, h, T, False, self.attn_dropout, self.training, bias=bias)
        return self.out(ctx.to(x.dtype), dropout_p=dropout_p, residual=residual)


class Wav2Vec2Encoder(nn.Module):
    """wav2vec 2.0 encoder: conv feature extractor -> LayerNorm -> projection -> time masking -> conv positions ->
    Transformer layers on packed frames.  ``layer_norm_first`` (the *large* recipe) uses pre-LN layers with a final
    LayerNorm, otherwise post-LN layers after an input LayerNorm."""

    def __init__(self, dim=1024, layers=24, heads=16, ffn=4096, dropout=0.1, attn_dropout=0.1, activation="gelu",
                 layer_norm_first=True, extractor_mode="layer_norm", conv_layers=W2V_LARGE_CONV, conv_bias=False,
                 mask_prob=0.0, mask_length=10, layerdrop=0.0, freeze_extractor=True, pos_kernel=128, pos_groups=16,
                 dropout_input=0.0, gated_relative_position=False, num_buckets=320, max_distance=800,
                 mask_channel_prob=0.0, mask_channel_length=64):
        super().__init__()
        # -wav2vec_spec_augment: spans of feature channels are zeroed per utterance during training (probability 0.2, span
        # 64; reference: onmt/models/speech_recognizer/wav2vec2.py:188-190 -> fairseq's mask_channel_*)
        self.mask_channel_prob, self.mask_channel_length = mask_channel_prob, mask_channel_length
        self.extractor = ConvFeatureExtractor(conv_layers, extractor_mode, conv_bias)
        self.freeze_extractor = freeze_extractor
        if freeze_extractor:
            for p in self.extractor.parameters():
                p.requires_grad_(False)
        self.feat_norm = nn.LayerNorm(self.extractor.out_dim)
        self.post_extract_proj = nn.Linear(self.extractor.out_dim, dim)
        self.dropout_input = dropout_input
        self.mask_emb = nn.Parameter(torch.empty(dim).uniform_())
        self.mask_prob, self.mask_length = mask_prob, mask_length
        self.pos_conv = ConvPositionalEmbedding(dim, pos_kernel, pos_groups)
        self.layer_norm_first = layer_norm_first
        self.input_norm = LayerNorm(dim)      # applied before the layers (post-LN recipe) or after them (pre-LN)
        self.layers = nn.ModuleList([
            EncoderLayer(dim, heads, ffn, dropout, attn_dropout, activation, attn_bias=True, death_rate=layerdrop,
                         post_norm=not layer_norm_first) for _ in range(layers)])
        if gated_relative_position:      # WavLM: every layer's attention gets the gated relative-position bias
            owner = None
            for layer in self.layers:
                layer.attn = GatedRelPosSelfAttention(dim, heads, attn_dropout, num_buckets, max_distance, table_owner=owner)
                owner = owner or layer.attn
        self.dim = dim
        self.adapters = None

    def add_adapters(self, n_languages: int, location: int = 1, downsample: int = 4):
        """``-wav2vec_adapter``: one bottleneck adapter per language in front of every Transformer layer (location 1; the
        layer's input becomes ``x + adapter_lang(x)``), chosen by the batch's source language
        (reference: onmt/models/speech_recognizer/fairseq_wav2vec2/wav2vec2.py:1112-1115, 1262-1280, 1494-1500)."""
        from .multilingual import MultilingualAdapter
        if location != 1:
            raise NotImplementedError("-wav2vec_adapter %d: only location 1 (in front of each layer) is built" % location)
        self.adapters = nn.ModuleList([MultilingualAdapter(self.dim, self.dim // downsample, n_languages) for _ in self.layers])

    def forward(self, source, lang: Optional[int] = None) -> Tuple[torch.Tensor, PackedSeqs]:
        if self.adapters is not None and lang is None:
            raise ValueError("this encoder has language adapters: the batch must carry its source language id")
        feats, lengths = split_audio_batch(source)
        wav = feats[:, :, 0].float()
        if self.freeze_extractor:
            with torch.no_grad():
                x = self.extractor(wav)
        else:
            x = self.extractor(wav)
        out_len = self.extractor.output_lengths(lengths).clamp(max=x.shape[1])
        x = self.post_extract_proj(self.feat_norm(x))
        if self.dropout_input > 0:
            x = F.dropout(x, self.dropout_input, self.training)
        B, T, _ = x.shape
        valid = torch.arange(T, device=x.device)[None, :] < out_len[:, None]
        if self.training and self.mask_prob > 0:
            m = compute_mask_spans(B, T, out_len.cpu(), self.mask_prob, self.mask_length).to(x.device)
            x = torch.where(m.unsqueeze(-1), self.mask_emb.to(x.dtype).expand_as(x), x)
        if self.training and self.mask_channel_prob > 0:
            full = torch.full((B,), x.shape[2], dtype=torch.long)
            cm = compute_mask_spans(B, x.shape[2], full, self.mask_channel_prob, self.mask_channel_length).to(x.device)
            x = x.masked_fill(cm.unsqueeze(1), 0.0)
        x = x * valid.unsqueeze(-1)
        x = x + self.pos_conv(x)
        packed, seqs = pack_padded(x, out_len)
        packed = packed.to(torch.bfloat16) if (packed.is_cuda and ops.fused_param(self.input_norm.weight)) else packed
        if not self.layer_norm_first:
            packed = self.input_norm(packed)
        for i, layer in enumerate(self.layers):
            if self.adapters is not None:
                packed = self.adapters[i](packed, lang)
            packed = layer(packed, seqs)
        if self.layer_norm_first:
            packed = self.input_norm(packed)
        return packed, seqs


class WhisperEncoder(nn.Module):
    """Whisper audio encoder: Conv1d(mels -> d, k3) + GELU, Conv1d(d -> d, k3, stride 2) + GELU, fixed sinusoidal
    positions, pre-LN layers, final LayerNorm.  Accepts any number of mel bins (the reference hard-codes 128 + 1)."""

    def __init__(self, n_mels=80, dim=1280, layers=32, heads=20, ffn=5120, max_positions=1500, dropout=0.0,
                 attn_dropout=0.0, layerdrop=0.0):
        super().__init__()
        self.conv1 = nn.Conv1d(n_mels, dim, 3, padding=1)
        self.conv2 = nn.Conv1d(dim, dim, 3, stride=2, padding=1)
        self.register_buffer("positions", sinusoidal_table(max_positions, dim), persistent=False)
        self.layers = nn.ModuleList([EncoderLayer(dim, heads, ffn, dropout, attn_dropout, "gelu", attn_bias=True,
                                                  death_rate=layerdrop) for _ in range(layers)])
        self.final_norm = LayerNorm(dim)
        self.n_mels, self.dim = n_mels, dim

    def forward(self, source):
        feats, lengths = split_audio_batch(source)           # [B, T, n_mels]
        assert feats.shape[-1] == self.n_mels, "expected %d mel bins (+1 padding channel), got %d" % (self.n_mels, feats.shape[-1])
        if feats.is_cuda and ops.fused_param(self.conv1.weight) and self.n_mels % 8 == 0:
            from ..ops.conv import conv1d                       # both stem layers as GEMMs with GELU in the epilogue
            x = conv1d(feats, self.conv1.weight, self.conv1.bias, 1, "gelu", padding=1)
            x = conv1d(x, self.conv2.weight, self.conv2.bias, 2, "gelu", padding=1)
        else:
            x = F.gelu(self.conv1(feats.transpose(1, 2).float()))
            x = F.gelu(self.conv2(x)).transpose(1, 2)             # [B, T/2, d]
        out_len = torch.div(lengths + 1, 2, rounding_mode="floor").clamp(max=x.shape[1])
        if x.shape[1] > self.positions.shape[0]:
            self.positions = sinusoidal_table(x.shape[1], self.dim).to(x.device)
        x = x + self.positions[:x.shape[1]].to(x.dtype)
        packed, seqs = pack_padded(x, out_len)
        packed = packed.to(torch.bfloat16) if (packed.is_cuda and ops.fused_param(self.final_norm.weight)) else packed
        for layer in self.layers:
            packed = layer(packed, seqs)
        return self.final_norm(packed), seqs


class SpeechTransformerEncoder(nn.Module):
    """Filterbank encoder of the ``speech_transformer`` family: linear projection of (stacked) frames, or two
    stride-2 Conv2d layers (x4 subsampling) followed by a projection, then sinusoidal positions and pre-LN layers."""

    def __init__(self, opt, input_size: int):
        super().__init__()
        dim = opt.model_size
        self.cnn = bool(getattr(opt, "cnn_downsampling", False))
        self.channels = getattr(opt, "upsampling", 1) if False else 1
        if self.cnn:
            # -no_batch_norm: the two convolutions without BatchNorm2d (reference: onmt/models/transformers.py:100-105)
            bn = (lambda: [nn.BatchNorm2d(32)]) if not getattr(opt, "no_batch_norm", False) else (lambda: [])
            self.conv = nn.Sequential(nn.Conv2d(1, 32, 3, stride=2, padding=1), nn.ReLU(), *bn(),
                                      nn.Conv2d(32, 32, 3, stride=2, padding=1), nn.ReLU(), *bn())
            feat = ((input_size + 1) // 2 + 1) // 2 * 32
            self.proj = nn.Linear(feat, dim)
        else:
            self.proj = nn.Linear(input_size, dim)
        n = opt.encoder_layers if getattr(opt, "encoder_layers", -1) > 0 else opt.layers
        self.register_buffer("positions", sinusoidal_table(getattr(opt, "max_position_length", 2048), dim), persistent=False)
        self.layers = nn.ModuleList([EncoderLayer(dim, opt.n_heads, opt.inner_size, opt.dropout, opt.attn_dropout,
                                                  opt.ffn_activation) for _ in range(n)])
        self.final_norm = LayerNorm(dim)
        self.emb_dropout = opt.emb_dropout
        self.dim = dim
        # -no_input_scale: projected frames are not multiplied by sqrt(model size) before the positions are added
        # (reference: onmt/models/speech_recognizer/relative_transformer.py:49, 167)
        self.input_scale = 1.0 if getattr(opt, "no_input_scale", False) else math.sqrt(dim)
        # -multilingual_linear_projection: the encoder output goes through one square matrix per source language
        # (reference: onmt/models/speech_recognizer/relative_transformer.py:72-76, 232-237)
        self.linear_proj = None
        if getattr(opt, "multilingual_linear_projection", False):
            n = max(1, int(getattr(opt, "n_languages", 1) or 1))
            self.linear_proj = nn.Parameter(torch.randn(n, dim, dim) * math.sqrt(2.0 / (dim + dim)))

    def forward(self, source, lang=None):
        feats, lengths = split_audio_batch(source)
        if self.cnn:
            x = self.conv(feats.unsqueeze(1).float())                     # [B, 32, T/4, F/4]
            x = x.permute(0, 2, 1, 3).reshape(x.shape[0], x.shape[2], -1)
            lengths = torch.div(torch.div(lengths + 1, 2, rounding_mode="floor") + 1, 2, rounding_mode="floor")
        else:
            x = feats.float()
        x = self.proj(x) * self.input_scale
        if x.shape[1] > self.positions.shape[0]:
            self.positions = sinusoidal_table(x.shape[1], self.dim).to(x.device)
        x = x + self.positions[:x.shape[1]].to(x.dtype)
        x = F.dropout(x, self.emb_dropout, self.training)
        packed, seqs = pack_padded(x, lengths.clamp(max=x.shape[1]))
        packed = packed.to(torch.bfloat16) if (packed.is_cuda and ops.fused_param(self.final_norm.weight)) else packed
        for layer in self.layers:
            packed = layer(packed, seqs)
        out = self.final_norm(packed)
        if self.linear_proj is not None:
            if lang is None:
                raise ValueError("-multilingual_linear_projection needs the source language id of the batch")
            out = out @ self.linear_proj[int(lang)].to(out.dtype)
        return out, seqs
