"""Builders that assemble the typed blocks into the NLLB (dense 600M / 1B / 3B) and LLaMA / LLaMA-2 architectures,
with randomly initialised weights and helpers to map fairseq2-style checkpoint keys.

Reference: onmt/models/nllb/nllb_builder.py:27-260 (``NllbConfig``, ``NllbBuilder``),
onmt/models/llama2/builder.py:38-430 (``LLaMAConfig``, ``LLaMABuilder``, ``convert_model_state_dict``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .blocks import (GLUFeedForwardNetwork, Linear, RMSNorm, RotaryEncoder, SinusoidalPositionEncoder, StandardEmbedding,
                     StandardFeedForwardNetwork, StandardMultiheadAttention, StandardTransformerDecoder,
                     StandardTransformerDecoderLayer, StandardTransformerEncoder, StandardTransformerEncoderLayer,
                     TiedProjection, TransformerDecoderModel, TransformerEmbeddingFrontend, TransformerModel, TransformerNormOrder)

__all__ = ["NllbConfig", "NllbBuilder", "create_nllb_model", "nllb_archs", "LLaMAConfig", "LLaMABuilder", "create_llama_model",
           "llama_archs", "convert_llama_state_dict"]


@dataclass
class NllbConfig:
    model_dim: int = 1024
    max_seq_len: int = 1024
    vocabulary_size: int = 256206
    pad_idx: Optional[int] = 1
    num_encoder_layers: int = 24
    num_decoder_layers: int = 24
    num_encoder_attn_heads: int = 16
    num_decoder_attn_heads: int = 16
    ffn_inner_dim: int = 1024 * 8
    dropout_p: float = 0.1


nllb_archs = {
    "dense_600m": lambda: NllbConfig(model_dim=1024, num_encoder_layers=12, num_decoder_layers=12, ffn_inner_dim=1024 * 4),
    "dense_1b": lambda: NllbConfig(model_dim=1024, num_encoder_layers=24, num_decoder_layers=24, ffn_inner_dim=1024 * 8),
    "dense_3b": lambda: NllbConfig(model_dim=2048, num_encoder_layers=24, num_decoder_layers=24, ffn_inner_dim=1024 * 8),
}


class NllbBuilder:
    """Override the ``build_*`` methods to change a part of the architecture."""

    def __init__(self, config: NllbConfig):
        self.config = config

    def build_embedding(self):
        c = self.config
        return StandardEmbedding(c.vocabulary_size, c.model_dim, c.pad_idx, scaled=True)

    def build_frontend(self, embed):
        c = self.config
        pos = SinusoidalPositionEncoder(c.model_dim, c.max_seq_len, legacy_pad_idx=c.pad_idx)
        return TransformerEmbeddingFrontend(embed, pos, dropout_p=c.dropout_p)

    def build_attention(self, num_heads, static_kv=False):
        c = self.config
        return StandardMultiheadAttention(c.model_dim, num_heads, attn_dropout_p=c.dropout_p, static_kv=static_kv)

    def build_ffn(self):
        c = self.config
        return StandardFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, norm_order=TransformerNormOrder.PRE)

    def build_encoder(self):
        c = self.config
        layers = [StandardTransformerEncoderLayer(self.build_attention(c.num_encoder_attn_heads), self.build_ffn(), c.model_dim,
                                                  c.dropout_p, TransformerNormOrder.PRE) for _ in range(c.num_encoder_layers)]
        return StandardTransformerEncoder(layers, c.model_dim, TransformerNormOrder.PRE)

    def build_decoder(self):
        c = self.config
        layers = [StandardTransformerDecoderLayer(self.build_attention(c.num_decoder_attn_heads),
                                                  self.build_attention(c.num_decoder_attn_heads, static_kv=True), self.build_ffn(),
                                                  c.model_dim, c.dropout_p, TransformerNormOrder.PRE)
                  for _ in range(c.num_decoder_layers)]
        return StandardTransformerDecoder(layers, c.model_dim, TransformerNormOrder.PRE)

    def build_model(self) -> TransformerModel:
        embed = self.build_embedding()
        return TransformerModel(self.build_frontend(embed), self.build_encoder(), self.build_frontend(embed), self.build_decoder(),
                                TiedProjection(embed.weight), self.config.pad_idx)


def create_nllb_model(config_or_arch="dense_600m", device=None, dtype=None) -> TransformerModel:
    cfg = nllb_archs[config_or_arch]() if isinstance(config_or_arch, str) else config_or_arch
    model = NllbBuilder(cfg).build_model()
    return model.to(device=device, dtype=dtype) if (device or dtype) else model


@dataclass
class LLaMAConfig:
    model_dim: int = 4096
    max_seq_len: int = 2048
    vocabulary_size: int = 32000
    num_layers: int = 32
    num_attn_heads: int = 32
    num_key_value_heads: int = 32
    ffn_inner_dim: int = 4096 * 4
    ffn_inner_dim_to_multiple: int = 256
    dropout_p: float = 0.1


llama_archs = {
    "7b": lambda: LLaMAConfig(),
    "13b": lambda: LLaMAConfig(model_dim=5120, num_layers=40, num_attn_heads=40, num_key_value_heads=40, ffn_inner_dim=5120 * 4),
    "33b": lambda: LLaMAConfig(model_dim=6656, num_layers=60, num_attn_heads=52, num_key_value_heads=52, ffn_inner_dim=6656 * 4),
    "65b": lambda: LLaMAConfig(model_dim=8192, num_layers=80, num_attn_heads=64, num_key_value_heads=64, ffn_inner_dim=8192 * 4),
    "llama2_7b": lambda: LLaMAConfig(max_seq_len=4096),
    "llama2_13b": lambda: LLaMAConfig(model_dim=5120, max_seq_len=4096, num_layers=40, num_attn_heads=40, num_key_value_heads=40,
                                      ffn_inner_dim=5120 * 4),
    "llama2_70b": lambda: LLaMAConfig(model_dim=8192, max_seq_len=4096, num_layers=80, num_attn_heads=64, num_key_value_heads=8,
                                      ffn_inner_dim=int(8192 * 4 * 1.3), ffn_inner_dim_to_multiple=4096),
}


class LLaMABuilder:
    def __init__(self, config: LLaMAConfig):
        self.config = config
        self.pos_encoder = RotaryEncoder(config.model_dim // config.num_attn_heads, config.max_seq_len)

    def build_layer_norm(self, dim):
        return RMSNorm(dim, eps=1e-5)

    def build_attention(self):
        c = self.config
        return StandardMultiheadAttention(c.model_dim, c.num_attn_heads, c.num_key_value_heads, self.pos_encoder, bias=False,
                                          attn_dropout_p=c.dropout_p)

    def build_ffn(self):
        c = self.config
        return GLUFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=False, inner_dim_to_multiple=c.ffn_inner_dim_to_multiple)

    def build_decoder_layer(self):
        c = self.config
        return StandardTransformerDecoderLayer(self.build_attention(), None, self.build_ffn(), c.model_dim, c.dropout_p,
                                               TransformerNormOrder.PRE, self.build_layer_norm)

    def build_model(self) -> TransformerDecoderModel:
        c = self.config
        embed = StandardEmbedding(c.vocabulary_size, c.model_dim)
        frontend = TransformerEmbeddingFrontend(embed, None, no_scale=True, dropout_p=c.dropout_p)
        decoder = StandardTransformerDecoder([self.build_decoder_layer() for _ in range(c.num_layers)], c.model_dim,
                                             TransformerNormOrder.PRE, self.build_layer_norm)
        return TransformerDecoderModel(frontend, decoder, Linear(c.model_dim, c.vocabulary_size, bias=False))


def create_llama_model(config_or_arch="llama2_7b", device=None, dtype=None) -> TransformerDecoderModel:
    cfg = llama_archs[config_or_arch]() if isinstance(config_or_arch, str) else config_or_arch
    model = LLaMABuilder(cfg).build_model()
    return model.to(device=device, dtype=dtype) if (device or dtype) else model


_LLAMA_KEYS = {"tok_embeddings": "decoder_frontend.embed", "attention.wq": "self_attn.q_proj", "attention.wk": "self_attn.k_proj",
               "attention.wv": "self_attn.v_proj", "attention.wo": "self_attn.output_proj", "attention_norm": "self_attn_layer_norm",
               "feed_forward.w1": "ffn.gate_proj", "feed_forward.w2": "ffn.output_proj", "feed_forward.w3": "ffn.inner_proj",
               "ffn_norm": "ffn_layer_norm", "output": "final_proj"}


def convert_llama_state_dict(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Original LLaMA checkpoint keys (``layers.N.attention.wq.weight`` ...) -> keys of ``TransformerDecoderModel``."""
    out = {}
    for key, val in state.items():
        if key.endswith("rope.freqs"):
            continue
        new = key
        if new.startswith("layers."):
            new = "decoder." + new
        elif new.startswith("norm."):
            new = "decoder.layer_norm." + new[len("norm."):]
        for old, repl in _LLAMA_KEYS.items():
            parts = new.split(".")
            joined = ".".join(parts)
            if "." + old + "." in "." + joined:
                new = ("." + joined).replace("." + old + ".", "." + repl + ".")[1:]
                break
        out[new] = val
    return out
