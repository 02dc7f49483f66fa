"""Transformer-XL style relative-position models: ``relative_transformer`` (encoder-decoder), the Transformer-XL
language model, and streaming decoding with segment memories.

Relative self-attention: ``score(i, j) = (q_i + u) . k_j + (q_i + v) . r_{i-j}`` with sinusoidal (or learnable)
relative embeddings ``r`` projected per layer and the two global biases ``u = r_w_bias``, ``v = r_r_bias``; the
``BD`` term is computed against all distances and aligned with the classic relative shift.  The projections and the
FFN run on the fused GEMM path (packed rows); the score / shift / softmax part is evaluated per padded batch with
PyTorch ops (a tcgen05 kernel with the shift folded into the index math is not built yet).

Reference: onmt/modules/optimized/relative_self_attention_func.py:79-504, onmt/modules/relative_attention.py:7-504
(``_rel_shift`` :7), onmt/models/relative_transformer.py:52-1100 (encoder :52, decoder :295, ``StreamState`` :947),
onmt/models/transformer_xl.py:111.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import CrossAttention, Embedding, FeedForward, LayerNorm, Linear, PackedSeqs
from .transformer import DecodingState, Generator, Seq2SeqBase


def relative_sinusoid(positions: torch.Tensor, dim: int) -> torch.Tensor:
    """positions [L] (may be negative) -> [L, dim] = [sin | cos] with inverse frequencies 1 / 10000^(2i/dim)."""
    inv = 1.0 / (10000 ** (torch.arange(0.0, dim, 2.0, device=positions.device) / dim))
    ang = positions.float()[:, None] * inv[None, :]
    return torch.cat([ang.sin(), ang.cos()], dim=-1)


def rel_shift(x: torch.Tensor) -> torch.Tensor:
    """[..., Tq, L] scores against distances (Tq-1 ... -(Tk-1)) -> aligned so that column j is key j (first Tk columns)."""
    *lead, tq, L = x.shape
    x = F.pad(x, (1, 0))
    x = x.reshape(*lead, L + 1, tq)[..., 1:, :].reshape(*lead, tq, L)
    return x


class RelativeSelfAttention(nn.Module):
    def __init__(self, dim: int, heads: int, attn_dropout: float = 0.0, causal: bool = False, learnable_pos: bool = False,
                 max_len: int = 512):
        super().__init__()
        self.dim, self.heads, self.hd = dim, heads, dim // heads
        self.qkv = Linear(dim, 3 * dim)
        self.pos = Linear(dim, dim, bias=False)
        self.out = Linear(dim, dim)
        self.r_w_bias = nn.Parameter(torch.zeros(heads, self.hd))
        self.r_r_bias = nn.Parameter(torch.zeros(heads, self.hd))
        nn.init.normal_(self.r_w_bias, 0, 0.02)
        nn.init.normal_(self.r_r_bias, 0, 0.02)
        self.attn_dropout, self.causal = attn_dropout, causal
        self.learnable_pos = learnable_pos
        if learnable_pos:
            self.pos_emb = nn.Parameter(torch.zeros(2 * max_len + 1, dim))
            nn.init.normal_(self.pos_emb, 0, 0.02)
            self.max_len = max_len

    def _positions(self, tq: int, tk: int, device):
        dist = torch.arange(tq - 1, -tk, -1, device=device)            # Tq-1 ... -(Tk-1)  (length Tq + Tk - 1)
        if self.learnable_pos:
            return self.pos_emb[(dist.clamp(-self.max_len, self.max_len) + self.max_len)]
        return relative_sinusoid(dist, self.dim)

    def forward(self, x, seqs: PackedSeqs, memory: Optional[torch.Tensor] = None, residual=None, dropout_p: float = 0.0):
        """x packed [N, H].  ``memory`` [B, M, H] (padded) is prepended to keys/values (streaming / Transformer-XL)."""
        H, h, d = self.dim, self.heads, self.hd
        qkv_packed = self.qkv(x)
        if ((memory is None or memory.shape[1] == 0) and qkv_packed.is_cuda and qkv_packed.dtype == torch.bfloat16 and d == 64
                and int(seqs.max_len) <= 128):
            # packed kernel: scores, relative shift (index arithmetic), softmax, dropout and value product per (sequence, head)
            from ..ops.rel_attention import rel_self_attention
            T = int(seqs.max_len)
            r = self.pos(self._positions(T, T, x.device).to(torch.bfloat16))
            ctx = rel_self_attention(qkv_packed, r.to(torch.bfloat16), self.r_w_bias, self.r_r_bias, seqs.cu, h, T, T - 1, self.causal,
                                     self.attn_dropout, self.training)
            return self.out(ctx, dropout_p=dropout_p, residual=residual)
        if (memory is None or memory.shape[1] == 0) and (getattr(self, "force_bias_path", False) or (
                qkv_packed.is_cuda and qkv_packed.dtype == torch.bfloat16 and d == 64)):
            return self.out(self._attend_with_bias(qkv_packed, seqs), dropout_p=dropout_p, residual=residual)
        qkv = seqs.pad(qkv_packed, time_first=False).float()          # [B, T, 3H]
        B, T, _ = qkv.shape
        q, k, v = qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:]
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
        key_valid = torch.arange(T, device=x.device)[None, :] < lengths[:, None]
        if memory is not None and memory.shape[1] > 0:
            mkv = self.qkv(memory.reshape(-1, H)).view(B, memory.shape[1], 3 * H).float()
            k = torch.cat([mkv[..., H:2 * H], k], 1)
            v = torch.cat([mkv[..., 2 * H:], v], 1)
            key_valid = torch.cat([torch.ones(B, memory.shape[1], dtype=torch.bool, device=x.device), key_valid], 1)
        Tk = k.shape[1]
        M = Tk - T
        r = self.pos(self._positions(T + M, Tk, x.device).to(x.dtype)).float()   # [T+M+Tk-1, H]
        q = q.view(B, T, h, d)
        k = k.view(B, Tk, h, d)
        v = v.view(B, Tk, h, d)
        r = r.view(-1, h, d)
        ac = torch.einsum("bqhd,bkhd->bhqk", q + self.r_w_bias.float(), k)
        # distances for query i (absolute position M + i) and key j: (M + i) - j; build BD for "virtual" queries 0..T+M-1
        bd_all = torch.einsum("bqhd,lhd->bhql", F.pad(q, (0, 0, 0, 0, M, 0)) + self.r_r_bias.float(), r)
        bd = rel_shift(bd_all)[..., M:, :Tk]
        s = (ac + bd) * (d ** -0.5)
        s = s.masked_fill(~key_valid[:, None, None, :], float("-inf"))
        if self.causal:
            tri = torch.ones(T, Tk, dtype=torch.bool, device=x.device).tril(diagonal=M)
            s = s.masked_fill(~tri[None, None], float("-inf"))
        p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0)
        p = F.dropout(p, self.attn_dropout, self.training)
        ctx = torch.einsum("bhqk,bkhd->bqhd", p, v).reshape(B, T, H).to(x.dtype)
        from ..ops.reference import unpad_packed
        ctx_packed = unpad_packed(ctx, seqs.cu, x.shape[0])
        return self.out(ctx_packed, dropout_p=dropout_p, residual=residual)


    def _attend_with_bias(self, qkv_packed, seqs: PackedSeqs):
        """Sequences longer than one tile on the tensor-core path: everything of the score that is not ``q . k`` - the
        content bias ``u . k_j`` and the shifted position term ``(q_i + v) . r_{i-j}`` - is one additive operand
        ``[B, h, T, T]`` of the packed attention kernels; its gradient comes back from the kernels and flows on to the
        queries, keys, position projection and both biases through these few PyTorch ops."""
        H, h, d = self.dim, self.heads, self.hd
        T = int(seqs.max_len)
        pad = seqs.pad(qkv_packed[:, :2 * H], time_first=False)                    # [B, T, 2H]
        B = pad.shape[0]
        q = pad[..., :H].float().view(B, T, h, d)
        k = pad[..., H:].float().view(B, T, h, d)
        r = self.pos(self._positions(T, T, qkv_packed.device).to(qkv_packed.dtype)).float().view(-1, h, d)   # [2T - 1, h, d]
        bd = rel_shift(torch.einsum("bqhd,lhd->bhql", q + self.r_r_bias.float(), r))[..., :T]
        uk = torch.einsum("hd,bkhd->bhk", self.r_w_bias.float(), k)[:, :, None, :]
        bias = (bd + uk) * (d ** -0.5)
        return ops.self_attention(qkv_packed, seqs.cu, h, T, self.causal, self.attn_dropout, self.training, bias=bias)


class RelativeEncoderLayer(nn.Module):
    def __init__(self, opt, causal=False):
        super().__init__()
        self.attn_norm = LayerNorm(opt.model_size)
        # -max_pos_length: relative distances beyond it share the outermost learnable position vector
        self.attn = RelativeSelfAttention(opt.model_size, opt.n_heads, opt.attn_dropout, causal,
                                          getattr(opt, "learnable_position_encoding", False),
                                          max_len=int(getattr(opt, "max_pos_length", 512) or 512))
        self.ffn_norm = LayerNorm(opt.model_size)
        self.ffn = FeedForward(opt.model_size, opt.inner_size, opt.dropout, opt.ffn_activation)
        self.dropout = opt.dropout

    def forward(self, x, seqs, memory=None):
        x = self.attn(self.attn_norm(x), seqs, memory, residual=x, dropout_p=self.dropout)
        return self.ffn(self.ffn_norm(x), residual=x, dropout_p=self.dropout)


class RelativeDecoderLayer(RelativeEncoderLayer):
    def __init__(self, opt, ignore_source=False):
        super().__init__(opt, causal=True)
        self.ignore_source = ignore_source
        if not ignore_source:
            self.cross_norm = LayerNorm(opt.model_size)
            self.cross_attn = CrossAttention(opt.model_size, opt.n_heads, opt.attn_dropout)

    def forward(self, x, seqs, context=None, src=None, memory=None):
        x = self.attn(self.attn_norm(x), seqs, memory, residual=x, dropout_p=self.dropout)
        if not self.ignore_source:
            x = self.cross_attn(self.cross_norm(x), seqs, context, src, residual=x, dropout_p=self.dropout)
        return self.ffn(self.ffn_norm(x), residual=x, dropout_p=self.dropout)


class RelativeTransformerEncoder(nn.Module):
    def __init__(self, opt, embed: Embedding):
        super().__init__()
        n = opt.encoder_layers if getattr(opt, "encoder_layers", -1) > 0 else opt.layers
        self.embed = embed
        self.layers = nn.ModuleList([RelativeEncoderLayer(opt) for _ in range(n)])
        self.final_norm = LayerNorm(opt.model_size)
        self.emb_dropout = opt.emb_dropout

    def forward(self, src: PackedSeqs):
        x = self.embed(src, self.emb_dropout)
        for layer in self.layers:
            x = layer(x, src)
        return self.final_norm(x)


class StreamState:
    """Per-layer hidden-state memories carried across segments (Transformer-XL recurrence / streaming decoding)."""

    def __init__(self, n_layers: int, max_memory: int):
        self.mems: List[Optional[torch.Tensor]] = [None] * n_layers
        self.max_memory = max_memory

    def update(self, layer: int, hidden_padded: torch.Tensor):
        prev = self.mems[layer]
        cat = hidden_padded.detach() if prev is None else torch.cat([prev, hidden_padded.detach()], 1)
        self.mems[layer] = cat[:, -self.max_memory:] if self.max_memory > 0 else None


class RelativeTransformerDecoder(nn.Module):
    def __init__(self, opt, embed: Embedding, ignore_source=False):
        super().__init__()
        self.embed = embed
        self.layers = nn.ModuleList([RelativeDecoderLayer(opt, ignore_source) for _ in range(opt.layers)])
        self.final_norm = LayerNorm(opt.model_size)
        self.emb_dropout = opt.emb_dropout

    def forward(self, tgt: PackedSeqs, context=None, src=None, stream: Optional[StreamState] = None):
        x = self.embed(tgt, self.emb_dropout)
        for i, layer in enumerate(self.layers):
            mem = stream.mems[i] if stream is not None else None
            if stream is not None:
                stream.update(i, tgt.pad(x, time_first=False))
            x = layer(x, tgt, context, src, mem)
        return self.final_norm(x)

    def step(self, tokens, position: int, state: DecodingState):
        """Incremental decoding re-runs the relative attention over the (short) prefix kept in the state."""
        B = tokens.shape[0]
        hist = state.buffers[0].get("tokens")
        hist = tokens[:, None] if hist is None else torch.cat([hist, tokens[:, None]], 1)
        for buf in state.buffers:
            buf["tokens"] = hist
        T = hist.shape[1]
        seqs = PackedSeqs.from_padded(hist, torch.full((B,), T, device=tokens.device))
        lengths = (~state.src_pad_mask).sum(1)
        from .layers import pack_padded
        ctx, src = pack_padded(state.context, lengths)
        x = self.forward(seqs, ctx, src)
        return x.view(B, T, -1)[:, -1]


class RelativeTransformer(Seq2SeqBase):
    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        pad = getattr(opt, "pad_idx", 0)
        # -absolute_position_encoding: sinusoidal absolute positions are added to the embeddings on top of the relative
        # attention (reference: onmt/models/multilingual_translator/relative_transformer.py:43, 54)
        absolute = bool(getattr(opt, "absolute_position_encoding", False))
        tgt_embed = Embedding(dicts["tgt"].size(), opt.model_size, pad, use_pos=absolute)
        src_embed = Embedding(dicts["src"].size(), opt.model_size, pad, use_pos=absolute)
        if getattr(opt, "join_embedding", False):
            src_embed.weight = tgt_embed.weight
        self.encoder = RelativeTransformerEncoder(opt, src_embed)
        self.decoder = RelativeTransformerDecoder(opt, tgt_embed)
        self.generator = Generator(opt.model_size, dicts["tgt"].size())
        if getattr(opt, "tie_weights", False):
            self.tie_weights()
        self.pad_idx, self.label_smoothing = pad, getattr(opt, "label_smoothing", 0.0)
        self.max_memory = getattr(opt, "max_memory_size", 0)

    def encode(self, batch):
        src = batch.packed_source()
        return self.encoder(src), src

    def init_stream(self):
        return StreamState(len(self.decoder.layers), self.max_memory)

    @torch.no_grad()
    def create_decoder_state(self, batch, beam_size: int = 1, **_unused):
        context, src = self.encode(batch)
        ctx = src.pad(context, time_first=False)
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        mask = torch.arange(ctx.shape[1], device=ctx.device)[None, :] >= lengths[:, None]
        return DecodingState(ctx, mask, len(self.decoder.layers), beam_size)


class TransformerXLLanguageModel(nn.Module):
    """Decoder-only LM with relative attention and segment-level recurrence (``train_language_model.py``)."""

    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        pad = getattr(opt, "pad_idx", 0)
        vocab = dicts["tgt"].size()
        self.decoder = RelativeTransformerDecoder(opt, Embedding(vocab, opt.model_size, pad, use_pos=False), ignore_source=True)
        self.generator = Generator(opt.model_size, vocab)
        self.generator.weight = self.decoder.embed.weight
        self.pad_idx, self.label_smoothing = pad, getattr(opt, "label_smoothing", 0.0)
        self.max_memory = getattr(opt, "max_memory_size", 0)
        apply_activation_layer(self, opt)

    def init_stream(self):
        return StreamState(len(self.decoder.layers), self.max_memory)

    def forward(self, batch, streaming_state: Optional[StreamState] = None, grad_scale=None, **_unused) -> Dict:
        tgt = batch.packed_target_input()
        labels = batch.packed_target_output()
        hidden = self.decoder(tgt, None, None, streaming_state)
        loss, correct, row_loss = ops.generator_cross_entropy(hidden, self.generator.weight, self.generator.bias, labels,
                                                              self.label_smoothing if self.training else 0.0, self.pad_idx,
                                                              grad_scale)
        return {"loss": loss, "correct": correct, "row_loss": row_loss, "hidden_packed": hidden, "tgt": tgt}


class MaxOutFeedForward(nn.Module):
    """``-activation_layer maxout``: the feed-forward block becomes one linear layer with ``ceil(inner / model)``
    candidates per output unit of which the largest is kept (reference: onmt/models/transformer_xl.py:44-46)."""

    def __init__(self, dim: int, inner: int):
        super().__init__()
        from .efficient_attention import MaxOut
        self.maxout = MaxOut(dim, dim, max(1, math.ceil(inner / dim)))

    def forward(self, x, residual=None, dropout_p: float = 0.0):
        y = self.maxout(x.float()).to(x.dtype)
        y = F.dropout(y, dropout_p, self.training) if dropout_p > 0 else y
        return y if residual is None else residual + y


def apply_activation_layer(model, opt):
    """``-activation_layer``: ``linear_relu_linear`` (default), ``linear_swish_linear`` (SiLU between the two linear
    layers) or ``maxout`` for the feed-forward blocks of the Transformer-XL language model."""
    kind = getattr(opt, "activation_layer", "linear_relu_linear") or "linear_relu_linear"
    if kind == "linear_relu_linear":
        return
    if kind not in ("linear_swish_linear", "maxout"):
        raise NotImplementedError("-activation_layer %s (known: linear_relu_linear, linear_swish_linear, maxout)" % kind)
    for layer in model.decoder.layers:
        if kind == "maxout":
            layer.ffn = MaxOutFeedForward(opt.model_size, opt.inner_size)
        else:
            layer.ffn = FeedForward(opt.model_size, opt.inner_size, opt.dropout, "silu")


def _xl_log_probs(self, tokens_tb):
    """Next-token log-probabilities ``[T, B, V]`` of a prefix matrix ``[T, B]`` (every column is a full-length prefix);
    what ``FusionNetwork`` asks of its language model."""
    T, B = tokens_tb.shape
    seqs = PackedSeqs.from_padded(tokens_tb.t().contiguous(), torch.full((B,), T, dtype=torch.int64, device=tokens_tb.device),
                                  pad_idx=self.pad_idx)
    with torch.no_grad():
        hidden = self.decoder(seqs, None, None, None)
        logits = self.generator(hidden).float()
    return torch.log_softmax(logits, -1).view(B, T, -1).transpose(0, 1)


TransformerXLLanguageModel.log_probs = _xl_log_probs


def register_builders(register):
    register("relative_transformer")(lambda opt, dicts: RelativeTransformer(opt, dicts))
    register("transformer_xl_lm", "TransformerXL", "transformer_xl")(lambda opt, dicts: TransformerXLLanguageModel(opt, dicts))
