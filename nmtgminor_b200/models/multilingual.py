"""Multilingual translation models (``-model multilingual_translator`` / ``translator``): language embeddings added to the
token embeddings, language-factorised weights (MFW: every Linear weight is modulated by a per-language rank-r outer
product, ``W_l = W * (r_l s_l^T) + (rm_l sm_l^T)``), language-specific LayerNorm, and bottleneck adapters per language.

Reference: onmt/models/multilingual_translator/relative_transformer.py:33,178, relative_transformer_layers.py,
onmt/modules/multilingual_factorized/* (``MFWPositionWiseFeedForward``, ``MFWEncdecMultiheadAttn``),
onmt/modules/multilingual_partitioned/*, onmt/modules/adaptive/*, onmt/modules/layer_norm.py (``MultilingualLayerNorm``),
pretrain_module/adapter.py:10,58.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Embedding, LayerNorm, PackedSeqs
from .transformer import Generator, Seq2SeqBase, TransformerDecoder, TransformerEncoder


class FactorizedLinear(nn.Module):
    """Linear layer whose weight is specialised per language by low-rank multiplicative and additive factors."""

    def __init__(self, d_in, d_out, n_languages, rank=1, bias=True, multiplicative=True, weight_drop=0.0, activation="none"):
        super().__init__()
        if activation not in ("none", "gelu", "silu"):
            raise NotImplementedError("-mfw_activation %s (none | gelu | silu)" % activation)
        # ``-weight_drop``: dropout on the shared weight (DropConnect); ``-mfw_activation``: non-linearity on the shared
        # weight after the multiplicative factors and before the additive ones
        # (reference: onmt/modules/multilingual_factorized/linear.py:70-103)
        self.weight_drop, self.activation = float(weight_drop), activation
        self.weight = nn.Parameter(torch.empty(d_out, d_in))
        nn.init.xavier_uniform_(self.weight)
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None
        self.r = nn.Parameter(torch.zeros(n_languages, rank, d_out))
        self.s = nn.Parameter(torch.zeros(n_languages, rank, d_in))
        nn.init.normal_(self.r, 0, 0.02)
        nn.init.normal_(self.s, 0, 0.02)
        self.multiplicative = multiplicative
        if multiplicative:
            self.rm = nn.Parameter(torch.ones(n_languages, 1, d_out))
            self.sm = nn.Parameter(torch.ones(n_languages, 1, d_in))

    def weight_for(self, lang: int):
        w = self.weight
        if self.weight_drop > 0:
            w = F.dropout(w, self.weight_drop, self.training)
        if self.multiplicative:
            w = w * (self.rm[lang].t() @ self.sm[lang])
        if self.activation == "gelu":
            w = F.gelu(w)
        elif self.activation == "silu":
            w = F.silu(w)
        return w + self.r[lang].t() @ self.s[lang]

    def forward(self, x, lang: int):
        return F.linear(x, self.weight_for(lang).to(x.dtype), self.bias.to(x.dtype) if self.bias is not None else None)


class PartitionedLinear(nn.Module):
    """Linear layer with partitioned weights (``-multilingual_partitioned_weights``): ``factor_size`` shared weight
    matrices, mixed per language by that language's factor vector - ``W(lang) = sum_f factor[lang, f] * W_f`` (and the
    same for the bias).  The factor table (an ``nn.Embedding(n_languages, factor_size)``) belongs to the model and is
    shared by every layer.  Reference: onmt/modules/multilingual_partitioned/linear.py:6-49, factor table in
    onmt/model_factory.py:480-482."""

    def __init__(self, d_in, d_out, factors: nn.Embedding):
        super().__init__()
        f = factors.embedding_dim
        self.d_in, self.d_out = d_in, d_out
        self.shared_weight = nn.Parameter(torch.empty(d_out * d_in, f))
        self.shared_bias = nn.Parameter(torch.zeros(d_out, f))
        nn.init.normal_(self.shared_weight, 0.0, (2.0 / (d_in + d_out)) ** 0.5)
        object.__setattr__(self, "_factors", factors)        # not a sub-module: the table is registered once, on the model

    def weight_for(self, lang: int):
        return torch.mv(self.shared_weight, self._factors.weight[lang]).view(self.d_out, self.d_in)

    def forward(self, x, lang: int):
        f = self._factors.weight[lang]
        w = torch.mv(self.shared_weight, f).view(self.d_out, self.d_in)
        return F.linear(x, w.to(x.dtype), torch.mv(self.shared_bias, f).to(x.dtype))


class MultilingualLayerNorm(nn.Module):
    def __init__(self, dim, n_languages, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n_languages, dim))
        self.bias = nn.Parameter(torch.zeros(n_languages, dim))
        self.eps = eps

    def forward(self, x, lang: int):
        return F.layer_norm(x, (x.shape[-1],), self.weight[lang].to(x.dtype), self.bias[lang].to(x.dtype), self.eps)


class _Norm(nn.Module):
    """LayerNorm, shared or per language (``-multilingual_layer_norm``)."""

    def __init__(self, dim, n_languages, per_language):
        super().__init__()
        self.norm = MultilingualLayerNorm(dim, n_languages) if per_language else LayerNorm(dim)
        self.per_language = per_language

    def forward(self, x, lang):
        return self.norm(x, lang) if self.per_language else self.norm(x)


class MFWLayer(nn.Module):
    """Encoder or decoder layer whose projections are language-factorised (``-multilingual_factorized_weights``):
    pre-LN self-attention [+ encoder-decoder attention] + feed-forward, every Linear a ``FactorizedLinear`` of rank
    ``-mfw_rank`` (additive factors, plus multiplicative ones unless switched off).  The attention cores run on the
    packed attention op; the projections are dense per-language weights applied with plain matrix products.
    Reference: onmt/models/multilingual_translator/relative_transformer_layers.py, onmt/modules/multilingual_factorized/*."""

    def __init__(self, opt, n_languages: int, decoder: bool, factors: Optional[nn.Embedding] = None):
        super().__init__()
        d, inner, r = opt.model_size, opt.inner_size, max(1, int(getattr(opt, "mfw_rank", 1)))
        bias = not getattr(opt, "mfw_no_bias", False)
        lin = (lambda i, o: PartitionedLinear(i, o, factors)) if factors is not None else lambda i, o: FactorizedLinear(i, o, n_languages, rank=r, bias=bias,
                                            multiplicative=bool(getattr(opt, "mfw_multiplicative", False)),
                                            weight_drop=float(getattr(opt, "weight_drop", 0.0) or 0.0),
                                            activation=str(getattr(opt, "mfw_activation", "none") or "none"))
        per_lang_norm = bool(getattr(opt, "multilingual_layer_norm", False))
        self.heads, self.dim, self.decoder = opt.n_heads, d, decoder
        self.dropout, self.attn_dropout, self.act = opt.dropout, opt.attn_dropout, opt.ffn_activation
        self.attn_norm, self.qkv, self.out = _Norm(d, n_languages, per_lang_norm), lin(d, 3 * d), lin(d, d)
        if decoder:
            self.cross_norm, self.q, self.kv, self.cross_out = _Norm(d, n_languages, per_lang_norm), lin(d, d), lin(d, 2 * d), lin(d, d)
        self.ffn_norm, self.fc1, self.fc2 = _Norm(d, n_languages, per_lang_norm), lin(d, inner), lin(inner, d)

    def _drop(self, y, residual):
        return residual + F.dropout(y.float(), self.dropout, self.training).to(residual.dtype)

    def forward(self, x, seqs: PackedSeqs, lang: int, memory=None, mem_seqs=None, mem_lang: int = 0):
        from .. import ops
        from ..ops.reference import _act
        h = self.attn_norm(x, lang)
        ctx = ops.self_attention(self.qkv(h, lang).contiguous(), seqs.cu, self.heads, seqs.max_len, self.decoder, self.attn_dropout,
                                 self.training)
        x = self._drop(self.out(ctx, lang), x)
        if self.decoder and memory is not None:
            h = self.cross_norm(x, lang)
            ctx = ops.cross_attention(self.q(h, lang).contiguous(), self.kv(memory, lang).contiguous(), seqs.cu, mem_seqs.cu, self.heads,
                                      seqs.max_len, mem_seqs.max_len, self.attn_dropout, self.training)
            x = self._drop(self.cross_out(ctx, lang), x)
        h = self.ffn_norm(x, lang)
        h = F.dropout(_act(self.fc1(h, lang).float(), ops.ACT_IDS[self.act]), self.dropout, self.training).to(x.dtype)
        return self._drop(self.fc2(h, lang), x)


class Adapter(nn.Module):
    """Bottleneck adapter: LayerNorm -> down -> ReLU -> up, added to its input."""

    def __init__(self, dim, bottleneck):
        super().__init__()
        self.norm = LayerNorm(dim)
        self.down, self.up = nn.Linear(dim, bottleneck), nn.Linear(bottleneck, dim)
        nn.init.zeros_(self.up.weight)
        nn.init.zeros_(self.up.bias)

    def forward(self, x):
        return x + self.up(F.relu(self.down(self.norm(x).float()))).to(x.dtype)


class MultilingualAdapter(nn.Module):
    def __init__(self, dim, bottleneck, n_languages):
        super().__init__()
        self.adapters = nn.ModuleList([Adapter(dim, bottleneck) for _ in range(n_languages)])

    def forward(self, x, lang: int):
        return self.adapters[lang](x)


class MultilingualTransformer(Seq2SeqBase):
    """Transformer with language embeddings (sum), optional per-language adapters after every layer and an optional
    factorised output projection."""

    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        n_lang = max(len(dicts.get("langs", {"src": 0, "tgt": 1})), 1)
        pad = getattr(opt, "pad_idx", 0)
        tgt_embed = Embedding(dicts["tgt"].size(), opt.model_size, pad)
        src_embed = Embedding(dicts["src"].size(), opt.model_size, pad)
        if getattr(opt, "join_embedding", False):
            src_embed.weight = tgt_embed.weight
        self.encoder = TransformerEncoder(opt, src_embed)
        self.decoder = TransformerDecoder(opt, tgt_embed)
        # language-factorised layers replace the plain ones on the side(s) that ask for them
        self.mfw_enc = bool(getattr(opt, "multilingual_factorized_weights", False))
        self.mfw_dec = self.mfw_enc or bool(getattr(opt, "multilingual_factorized_weights_decoder", False))
        factors = None
        if getattr(opt, "multilingual_partitioned_weights", False):
            # partitioned weights: every projection of both stacks is a per-language mixture of shared matrices
            self.factor_embeddings = nn.Embedding(n_lang, int(getattr(opt, "mpw_factor_size", 8) or 8))
            factors = self.factor_embeddings
            self.mfw_enc = self.mfw_dec = True
        if self.mfw_enc:
            self.encoder.layers = nn.ModuleList([MFWLayer(opt, n_lang, decoder=False, factors=factors) for _ in self.encoder.layers])
        if self.mfw_dec:
            self.decoder.layers = nn.ModuleList([MFWLayer(opt, n_lang, decoder=True, factors=factors) for _ in self.decoder.layers])
        # Where the language vector meets the sqrt(d) scaling of the word embeddings: the encoder scales the sum unless
        # -encoder_early_emb_scale, the decoder scales the words only unless -decoder_late_emb_scale
        # (reference: onmt/models/multilingual_translator/relative_transformer.py:113-152, 259-311)
        self.enc_lang_scale = 1.0 if getattr(opt, "encoder_early_emb_scale", False) else math.sqrt(opt.model_size)
        self.dec_lang_scale = math.sqrt(opt.model_size) if getattr(opt, "decoder_late_emb_scale", False) else 1.0
        self.lang_embed = nn.Embedding(n_lang, opt.model_size)
        nn.init.normal_(self.lang_embed.weight, 0, opt.model_size ** -0.5)
        self.generator = Generator(opt.model_size, dicts["tgt"].size())
        if getattr(opt, "tie_weights", False):
            self.tie_weights()
        bott = int(getattr(opt, "adapter_bottleneck_size", 0) or 0)
        self.use_adapters = bool(getattr(opt, "multilingual_adapter", False)) and bott > 0
        if self.use_adapters:
            self.enc_adapters = nn.ModuleList([MultilingualAdapter(opt.model_size, bott, n_lang) for _ in self.encoder.layers])
            self.dec_adapters = nn.ModuleList([MultilingualAdapter(opt.model_size, bott, n_lang) for _ in self.decoder.layers])
        self.pad_idx, self.label_smoothing = pad, getattr(opt, "label_smoothing", 0.0)

    def _lang(self, batch, key, default):
        t = batch.get(key)
        return int(t.view(-1)[0]) if t is not None and t.numel() else default

    def encode(self, batch):
        src = batch.packed_source()
        lang = self._lang(batch, "source_lang", 0)
        x = self.encoder.embed(src, self.encoder.emb_dropout)
        x = x + (self.lang_embed.weight[lang] * self.enc_lang_scale).to(x.dtype)
        for i, layer in enumerate(self.encoder.layers):
            x = layer(x, src, lang) if self.mfw_enc else layer(x, src)
            if self.use_adapters:
                x = self.enc_adapters[i](x, lang)
        return self.encoder.final_norm(x), src

    def _decode_prefix(self, tgt: PackedSeqs, memory, src: PackedSeqs, lang: int):
        """The decoder stack with everything that depends on the target language: language embedding, factorised or
        partitioned weights, adapters."""
        dec = self.decoder
        x = dec.embed(tgt, dec.emb_dropout if self.training else 0.0) + (self.lang_embed.weight[lang] * self.dec_lang_scale).to(memory.dtype)
        for i, layer in enumerate(dec.layers):
            x = layer(x, tgt, lang, memory, src) if self.mfw_dec else layer(x, tgt, memory, src)
            if self.use_adapters:
                x = self.dec_adapters[i](x, lang)
        return dec.final_norm(x)

    def forward(self, batch, **kw):
        lang = self._lang(batch, "target_lang", min(1, self.lang_embed.num_embeddings - 1))
        dec = self.decoder
        original = dec.forward
        dec.forward = lambda tgt, memory, src: self._decode_prefix(tgt, memory, src, lang)
        try:
            return super().forward(batch, **kw)
        finally:
            dec.forward = original

    # Decoding.  The incremental caches of the plain layers know nothing of the language embedding, the per-language
    # weights and the adapters, so every step runs the decoder over the whole prefix of every hypothesis with the same
    # code as training: quadratic in the output length, and exactly the model that was trained.
    supports_logits_step = False

    @torch.no_grad()
    def create_decoder_state(self, batch, beam_size: int = 1, **_unused):
        from .transformer import DecodingState
        context, src = self.encode(batch)
        ctx_padded = src.pad(context, time_first=False)
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)[:ctx_padded.shape[0]]
        pad_mask = torch.arange(ctx_padded.shape[1], device=ctx_padded.device)[None, :] >= lengths[:, None]
        state = DecodingState(ctx_padded, pad_mask, 0, beam_size)
        state.tgt_lang_id = self._lang(batch, "target_lang", min(1, self.lang_embed.num_embeddings - 1))
        return state

    @torch.no_grad()
    def step(self, input_t, state, logits_only: bool = False):
        from .layers import pack_padded
        rows, t = input_t.shape
        dev = input_t.device
        tgt = PackedSeqs(input_t.reshape(-1).long().contiguous(), torch.arange(t, device=dev).repeat(rows),
                         (torch.arange(rows + 1, device=dev, dtype=torch.int32) * t), t)
        memory, src = pack_padded(state.context, (~state.src_pad_mask).sum(-1))
        hidden = self._decode_prefix(tgt, memory, src, state.tgt_lang_id).view(rows, t, -1)[:, -1]
        logits = self.generator(hidden)
        state.position += 1
        if logits_only:
            return {"logits": logits, "hidden": hidden, "coverage": None}
        return {"log_prob": torch.log_softmax(logits.float(), dim=-1), "hidden": hidden, "coverage": None}


def register_builders(register):
    register("multilingual_translator", "translator")(lambda opt, dicts: MultilingualTransformer(opt, dicts))
