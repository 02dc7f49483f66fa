"""Building blocks that run on PACKED token matrices ``[tokens, hidden]`` (no padding anywhere).

Every block is a thin ``nn.Module`` holding parameters and calling the functional ops of
``nmtgminor_b200.ops``; on a CUDA device with a flat parameter store attached the ops are the sm_100a
kernels, otherwise their PyTorch restatements.  Sequences are described by ``PackedSeqs`` (cumulative
offsets), which is what the variable-length attention kernel consumes.

Functional counterparts in the reference: ``MultiHeadAttention`` (onmt/modules/attention.py:15-141),
``SelfMultiheadAttn`` / ``EncdecMultiheadAttn`` (onmt/modules/optimized/self_attention.py:21-147,
encdec_attention.py:10-156), ``FeedForward`` / ``PositionWiseFeedForward`` (onmt/modules/linear.py:123-160,
onmt/modules/optimized/feed_forward.py:13-207), ``PrePostProcessing``
(onmt/modules/pre_post_processing.py:10-82) and ``PositionalEncoding``
(onmt/models/transformer_layers.py:354-442).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


@dataclass
class PackedSeqs:
    """A batch of sequences stored back to back.

    tokens / positions: int64 ``[capacity]`` (rows past ``cu[-1]`` hold the padding id / position 0),
    cu: int32 ``[B + 1]`` cumulative lengths, max_len: host upper bound on the longest sequence.
    """
    tokens: torch.Tensor
    positions: torch.Tensor
    cu: torch.Tensor
    max_len: int
    lengths: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)

    @property
    def batch_size(self) -> int:
        return self.cu.numel() - 1

    def to(self, device, non_blocking=True):
        mv = lambda t: t.to(device, non_blocking=non_blocking) if isinstance(t, torch.Tensor) else t
        return PackedSeqs(mv(self.tokens), mv(self.positions), mv(self.cu), self.max_len, mv(self.lengths),
                          {k: mv(v) for k, v in self.extras.items()})

    @staticmethod
    def from_padded(tokens_bt: torch.Tensor, lengths: torch.Tensor, capacity: Optional[int] = None, pad_idx: int = 0):
        """Pack a right-padded ``[B, T]`` matrix given per-row lengths."""
        B, T = tokens_bt.shape
        lengths = lengths.to(torch.int64)
        total = int(lengths.sum())
        cap = capacity if capacity is not None else total
        ar = torch.arange(T, device=tokens_bt.device)
        mask = ar[None, :] < lengths[:, None]
        toks = tokens_bt.new_full((cap,), pad_idx)
        pos = tokens_bt.new_zeros((cap,))
        toks[:total] = tokens_bt[mask]
        pos[:total] = ar[None, :].expand(B, T)[mask]
        cu = torch.zeros(B + 1, dtype=torch.int32, device=tokens_bt.device)
        cu[1:] = torch.cumsum(lengths, 0).to(torch.int32)
        return PackedSeqs(toks, pos, cu, int(lengths.max()) if B else 0, lengths)

    def pad(self, x: torch.Tensor, time_first: bool = True):
        """Packed ``[tokens, ...]`` -> padded ``[T, B, ...]`` (or ``[B, T, ...]``)."""
        from ..ops.reference import pad_packed
        out, _ = pad_packed(x, self.cu, self.max_len)
        return out.transpose(0, 1).contiguous() if time_first else out


def sinusoidal_table(n_pos: int, dim: int) -> torch.Tensor:
    """tensor2tensor-style table: ``[sin(pos * w_i) | cos(pos * w_i)]`` with ``w_i = 10000^(-i/(dim/2-1))``."""
    half = dim // 2
    inc = math.log(10000.0) / max(half - 1, 1)
    inv = torch.exp(torch.arange(half, dtype=torch.float32) * -inc)
    ang = torch.arange(n_pos, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=1)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))
        self.eps = eps

    def forward(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps)

    def with_residual(self, x):
        """``(x, LN(x))``; use the first result as the residual of ``x + f(LN(x))`` so that backward sums the two
        gradient paths inside the LayerNorm kernel."""
        return ops.layer_norm_residual(x, self.weight, self.bias, self.eps)


class Linear(nn.Module):
    """Affine map on packed rows with an optional fused epilogue (activation, dropout, residual)."""

    def __init__(self, d_in: int, d_out: int, bias: bool = True, init_std: Optional[float] = None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(d_out, d_in))
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None
        if init_std is None:
            nn.init.xavier_uniform_(self.weight)
        else:
            nn.init.normal_(self.weight, 0.0, init_std)

    def forward(self, x, act="none", dropout_p=0.0, residual=None):
        q = getattr(self, "_int8", None)
        if q is not None and not self.training and not x.is_cuda:
            # CPU inference with dynamically quantised weights (``-dynamic_quantile 1``)
            from ..ops.reference import _act
            y = _act(q(x.float()), ops.ACT_IDS[act] if not isinstance(act, int) else act).to(x.dtype)
            return y if residual is None else y + residual
        return ops.linear(x, self.weight, self.bias, act, dropout_p, residual, self.training)


def quantize_linears_for_cpu(model: nn.Module) -> int:
    """Attach an int8 dynamically quantised twin (per-tensor weight scale, activations quantised on the fly) to every
    ``Linear`` of ``model`` for CPU inference; returns how many were converted.  The fp32 weights stay in place, so the
    model still runs on a GPU.  Counterpart of the reference's ``torch.quantization.quantize_dynamic`` call
    (onmt/inference/fast_translator.py:176-190)."""
    engines = torch.backends.quantized.supported_engines
    torch.backends.quantized.engine = "fbgemm" if "fbgemm" in engines else ("qnnpack" if "qnnpack" in engines else engines[-1])
    from torch.ao.nn.quantized.dynamic import Linear as QLinear
    n = 0
    for m in model.modules():
        if isinstance(m, Linear):
            ref = nn.Linear(m.weight.shape[1], m.weight.shape[0], bias=m.bias is not None)
            ref.weight.data = m.weight.detach().float().cpu()
            if m.bias is not None:
                ref.bias.data = m.bias.detach().float().cpu()
            ref.qconfig = torch.ao.quantization.default_dynamic_qconfig
            object.__setattr__(m, "_int8", QLinear.from_float(ref))      # not a registered sub-module: checkpoints are unchanged
            n += 1
    return n


class Embedding(nn.Module):
    """Token embedding * scale + (sinusoidal | learned) position row, then dropout, in one kernel."""

    def __init__(self, vocab: int, dim: int, pad_idx: int = 0, scale: Optional[float] = None, max_pos: int = 1024,
                 learned_pos: bool = False, pos_offset: int = 0, use_pos: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim))
        nn.init.normal_(self.weight, 0.0, dim ** -0.5)
        with torch.no_grad():
            self.weight[pad_idx].zero_()
        self.pad_idx = pad_idx
        self.scale = math.sqrt(dim) if scale is None else scale
        self.learned_pos = learned_pos
        self.pos_offset = pos_offset
        self.use_pos = use_pos
        if use_pos:
            if learned_pos:
                self.pos = nn.Parameter(torch.empty(max_pos + pos_offset, dim))
                nn.init.normal_(self.pos, 0.0, 0.02)
            else:
                self.register_buffer("pos", sinusoidal_table(max_pos, dim), persistent=False)
                self._pos_work = None

    def renew(self, n_pos: int):
        if self.use_pos and not self.learned_pos and n_pos > self.pos.shape[0]:
            self.pos = sinusoidal_table(n_pos, self.pos.shape[1]).to(self.pos.device)
            self._pos_work = None

    def _pos_table(self, device):
        if not self.use_pos:
            return None
        if self.learned_pos:
            return self.pos
        if device.type != "cuda":
            return self.pos
        if self._pos_work is None or self._pos_work.device != device:
            self._pos_work = self.pos.to(device=device, dtype=torch.bfloat16)
        return self._pos_work

    word_dropout = 0.0      # probability of dropping a whole vocabulary entry for one batch (training only)

    def forward(self, seqs: PackedSeqs, dropout_p: float = 0.0):
        pos = seqs.positions + self.pos_offset if (self.use_pos and self.pos_offset) else seqs.positions
        tokens, scale = seqs.tokens, self.scale
        if self.training and self.word_dropout > 0:
            from ..modules.dropout import word_dropout_tokens
            tokens, mult = word_dropout_tokens(tokens, self.weight.shape[0], self.word_dropout, self.pad_idx)
            scale = scale * mult
        return ops.embedding(tokens, self.weight, pos if self.use_pos else None, self._pos_table(seqs.tokens.device),
                             scale, dropout_p, self.training, self.pad_idx, pos_trainable=self.learned_pos)


def rotate_queries_and_keys(qkv, positions, heads: int, base: float = 10000.0):
    """Rotary position encoding on the fused projection ``qkv [N, 3 * heads * d]``: queries and keys of the token at
    position ``t`` are rotated by the angles ``t / base^(2i/d)`` (half-split layout: column ``i`` pairs with column
    ``i + d/2``), values are left alone.  Scores then depend on the distance between query and key only."""
    N, W3 = qkv.shape
    d = W3 // (3 * heads)
    inv = 1.0 / (base ** (torch.arange(0, d, 2, device=qkv.device, dtype=torch.float32) / d))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]                     # [N, d/2]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, None, :]
    t = qkv.view(N, 3, heads, d)
    qk = t[:, :2].float()
    half = torch.cat([-qk[..., d // 2:], qk[..., :d // 2]], -1)
    qk = (qk * cos + half * sin).to(qkv.dtype)
    return torch.cat([qk, t[:, 2:]], 1).view(N, W3)


class SelfAttention(nn.Module):
    """Fused-QKV self-attention sub-layer: ``residual + D(out(attn(qkv(x))))``.  ``rotary`` (set by
    ``-rotary_position_encoding`` on encoder stacks) rotates queries and keys by their positions first."""

    rotary = False

    def __init__(self, dim: int, heads: int, attn_dropout: float = 0.0, bias: bool = False, causal: bool = False):
        super().__init__()
        self.dim, self.heads, self.attn_dropout, self.causal = dim, heads, attn_dropout, causal
        self.register_buffer("favor_projection", None, persistent=False)
        self.qkv = Linear(dim, 3 * dim, bias=bias)
        self.out = Linear(dim, dim, bias=bias)

    def enable_favor(self, nb_features: int = 0, seed: int = 0):
        """``-favor_attention``: softmax attention is replaced by its FAVOR+ estimate (positive orthogonal random
        features, cost linear in the sequence length); the projections keep their weights.
        (reference: onmt/models/speech_recognizer/wav2vec2.py:192-197, fairseq_wav2vec2 ``favor=``)"""
        if self.causal:
            raise NotImplementedError("-favor_attention is built for encoder (bidirectional) attention")
        from .efficient_attention import gaussian_orthogonal_random_matrix
        d = self.dim // self.heads
        m = nb_features or max(1, int(d * math.log(d)))
        self.favor_projection = gaussian_orthogonal_random_matrix(m, d, torch.Generator().manual_seed(seed)).to(self.qkv.weight.device)

    def _favor_attend(self, qkv, seqs: PackedSeqs):
        from ..ops.reference import unpad_packed
        from .efficient_attention import softmax_kernel
        h, d = self.heads, self.dim // self.heads
        padded = seqs.pad(qkv, time_first=False).float()                              # [B, T, 3H], zero rows past each length
        B, T, _ = padded.shape
        q, k, v = padded.view(B, T, 3, h, d).permute(2, 0, 3, 1, 4)                   # [B, h, T, d]
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
        keep = (torch.arange(T, device=qkv.device)[None, :] < lengths[:, None])[:, None, :, None].float()
        qf = softmax_kernel(q, self.favor_projection, True)
        kf = softmax_kernel(k, self.favor_projection, False) * keep
        kv = torch.einsum("bhtm,bhtd->bhmd", kf, v * keep)
        num = torch.einsum("bhtm,bhmd->bhtd", qf, kv)
        den = torch.einsum("bhtm,bhm->bht", qf, kf.sum(2))
        ctx = (num / den.clamp_min(1e-6)[..., None]).transpose(1, 2).reshape(B, T, self.dim)
        return unpad_packed(ctx.to(qkv.dtype), seqs.cu, qkv.shape[0])

    def forward(self, x, seqs: PackedSeqs, residual=None, dropout_p: float = 0.0):
        qkv = self.qkv(x)
        if self.rotary:
            qkv = rotate_queries_and_keys(qkv, seqs.positions, self.heads)
        if self.favor_projection is not None:
            return self.out(self._favor_attend(qkv, seqs), dropout_p=dropout_p, residual=residual)
        ctx = ops.self_attention(qkv, seqs.cu, self.heads, seqs.max_len, self.causal, self.attn_dropout, self.training)
        return self.out(ctx, dropout_p=dropout_p, residual=residual)

    # -- incremental decoding: x [B, H] is ONE new position per hypothesis --------------------------
    def step(self, x, cache: dict, residual=None):
        if self.rotary:
            raise NotImplementedError("rotary positions are built for encoder stacks (no incremental step)")
        H, h = self.dim, self.heads
        qkv = self.qkv(x)
        q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
        B = x.shape[0]
        if _fused_decode(qkv, H, h) and cache.get("cap"):
            # preallocated [rows, cap, H] caches: append in place, attend with the single-query kernel
            pos = cache.get("pos", 0)
            if "k" not in cache:
                for name in ("k", "v", "k_spare", "v_spare"):
                    cache[name] = torch.empty(B, cache["cap"], H, dtype=qkv.dtype, device=qkv.device)
            pos_dev = cache.get("pos_dev")
            if pos_dev is not None:
                # the write position lives on the device (advanced once per step by the caller): graph-replayable
                ops.ext().cache_append(k, v, cache["k"], cache["v"], 0, pos_dev)
                ctx = ops.ext().decode_attn(q, cache["k"], cache["v"], None, cache["cap"], h, (H // h) ** -0.5, pos_dev, 1)
            else:
                ops.ext().cache_append(k, v, cache["k"], cache["v"], pos)
                ctx = ops.ext().decode_attn(q, cache["k"], cache["v"], None, pos + 1, h, (H // h) ** -0.5)
                cache["pos"] = pos + 1
            return self.out(ctx, residual=residual)
        if "k" not in cache:
            cache["k"], cache["v"] = k.view(B, 1, H), v.view(B, 1, H)
        else:
            cache["k"] = torch.cat([cache["k"], k.view(B, 1, H)], 1)
            cache["v"] = torch.cat([cache["v"], v.view(B, 1, H)], 1)
        ctx = _cached_attention(q, cache["k"], cache["v"], h, None)
        return self.out(ctx, residual=residual)


def _fused_decode(t, dim, heads) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and dim // heads == 64


class CrossAttention(nn.Module):
    """Encoder-decoder attention sub-layer with a fused key/value projection of the encoder states."""

    def __init__(self, dim: int, heads: int, attn_dropout: float = 0.0, bias: bool = False, kv_dim: Optional[int] = None):
        super().__init__()
        self.dim, self.heads, self.attn_dropout = dim, heads, attn_dropout
        self.q = Linear(dim, dim, bias=bias)
        self.kv = Linear(kv_dim or dim, 2 * dim, bias=bias)
        self.out = Linear(dim, dim, bias=bias)

    def forward(self, x, seqs: PackedSeqs, memory, mem_seqs: PackedSeqs, residual=None, dropout_p: float = 0.0):
        ctx = ops.cross_attention(self.q(x), self.kv(memory), seqs.cu, mem_seqs.cu, self.heads, seqs.max_len,
                                  mem_seqs.max_len, self.attn_dropout, self.training)
        return self.out(ctx, dropout_p=dropout_p, residual=residual)

    def precompute(self, memory_padded):
        """memory_padded [B, Ts, H] -> cached keys / values [B, Ts, H] for incremental decoding."""
        B, T, Hm = memory_padded.shape
        kv = self.kv(memory_padded.reshape(B * T, Hm)).view(B, T, 2 * self.dim)
        return kv[..., :self.dim].contiguous(), kv[..., self.dim:].contiguous()

    def step(self, x, cache: dict, mem_mask, residual=None):
        q = self.q(x)
        ck, cv = cache["c_k"], cache["c_v"]
        if "c_len" in cache and _fused_decode(q, self.dim, self.heads):
            # one cache row per sentence, shared by its hypotheses
            ctx = ops.ext().decode_attn(q, ck, cv, cache["c_len"], ck.shape[1], self.heads, (self.dim // self.heads) ** -0.5)
            return self.out(ctx, residual=residual)
        if ck.shape[0] != q.shape[0]:
            rep = q.shape[0] // ck.shape[0]
            ck, cv = ck.repeat_interleave(rep, 0), cv.repeat_interleave(rep, 0)
        ctx = _cached_attention(q, ck, cv, self.heads, mem_mask)
        return self.out(ctx, residual=residual)


def _cached_attention(q, k, v, heads, key_pad_mask):
    """Single-position attention over cached keys.  q [B, H]; k, v [B, T, H]; key_pad_mask [B, T] True = pad."""
    B, T, H = k.shape
    d = H // heads
    qh = q.view(B, heads, 1, d).float()
    kh = k.view(B, T, heads, d).permute(0, 2, 1, 3).float()
    vh = v.view(B, T, heads, d).permute(0, 2, 1, 3).float()
    s = torch.matmul(qh, kh.transpose(-1, -2)) * (d ** -0.5)
    if key_pad_mask is not None:
        s = s.masked_fill(key_pad_mask[:, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vh).reshape(B, H).to(q.dtype)


class FeedForward(nn.Module):
    """``residual + D(fc2(D(act(fc1(x)))))`` executed as two GEMMs with fused epilogues.  ``glu`` (``-ffn_glu``): fc1 is
    twice as wide and the hidden state is ``act(first half) * second half`` (reference:
    onmt/modules/optimized/feed_forward.py:181-184)."""

    def __init__(self, dim: int, inner: int, dropout: float = 0.0, activation: str = "relu", glu: bool = False):
        super().__init__()
        self.fc1 = Linear(dim, inner * (2 if glu else 1))
        self.fc2 = Linear(inner, dim)
        self.dropout = dropout
        self.activation = activation
        self.glu = glu

    # -weight_drop p: DropConnect - dropout on both weight matrices during training
    # (reference: onmt/modules/optimized/feed_forward.py:30-40).  The masked weights exist for one step only, so this
    # path runs as plain matrix products instead of the fused feed-forward.
    weight_drop = 0.0

    def forward(self, x, residual=None, dropout_p: float = 0.0):
        if self.weight_drop > 0 and self.training:
            if self.glu:
                raise NotImplementedError("-weight_drop with -ffn_glu")
            from ..ops import reference as ref
            w1 = F.dropout(self.fc1.weight, self.weight_drop, True)
            w2 = F.dropout(self.fc2.weight, self.weight_drop, True)
            h = ref.linear(x, w1, self.fc1.bias, ops.ACT_IDS[self.activation], self.dropout, None)
            return ref.linear(h, w2, self.fc2.bias, 0, dropout_p, residual)
        if self.glu:
            h, gate = self.fc1(x).chunk(2, dim=-1)
            from ..ops.reference import _act
            h = (_act(h.float(), ops.ACT_IDS[self.activation]) * gate.float()).to(x.dtype)
            h = ops.dropout_add(h.contiguous(), None, self.dropout, self.training)
            return self.fc2(h, dropout_p=dropout_p, residual=residual)
        return ops.mlp(x, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias, self.activation, self.dropout,
                       dropout_p, residual, self.training)


def _sub(layer, fn, inp, residual, p, seqs, *args):
    """Sub-layer output + residual.  Element-wise dropout rides in the producing kernel; with ``layer.variational``
    the mask is shared along time instead and applied outside the kernel."""
    kw = {"seqs": seqs} if getattr(fn, "wants_seqs", False) else {}    # batch-ensemble blocks pick a member per sentence
    if getattr(layer, "variational", False) and layer.training and p > 0:
        from ..modules.dropout import variational_dropout
        y = fn(inp, *args, residual=None, dropout_p=0.0, **kw)
        return residual + variational_dropout(y, p, True, cu=seqs.cu)
    return fn(inp, *args, residual=residual, dropout_p=p, **kw)


def _scaled_sub(layer, fn, inp, residual, p, seqs, *args, scale=None):
    """``residual + scale * D(fn(inp))`` with ``scale`` a float (the half steps of a macaron block) or a learned scalar
    (``-rezero``: starts at zero, no LayerNorm in front).  Outside the fused residual epilogue, which cannot scale."""
    kw = {"seqs": seqs} if getattr(fn, "wants_seqs", False) else {}
    y = fn(inp, *args, residual=None, dropout_p=p, **kw)
    return residual + (y.float() * scale).to(y.dtype)


class _LayerOptions:
    """Structure switches shared by encoder and decoder layers (reference: onmt/models/transformer_layers.py:83-351):
    ``post_norm`` LayerNorm after the residual sum, ``rezero`` learned residual gates instead of LayerNorm
    (pre_post_processing.py:77-80), ``macaron`` an extra feed-forward half step in front of the attention with both
    feed-forward blocks scaled by 1/2, ``glu`` gated feed-forward."""

    def _init_options(self, dim, inner, fd, activation, post_norm, rezero, macaron, glu):
        self.post_norm, self.rezero, self.macaron = post_norm, rezero, macaron
        self.ffn_scale = 0.5 if macaron else None
        if macaron:
            self.mcr_norm = LayerNorm(dim)
            self.mcr_ffn = FeedForward(dim, inner, fd, activation, glu=glu)
        if rezero:
            # one residual gate per sub-layer: 0 self-attention, 1 feed-forward, 2 macaron feed-forward,
            # 3 encoder-decoder attention, 4 interleaved feed-forward (unused entries stay at zero)
            self.gates = nn.Parameter(torch.zeros(5))

    # -stochastic_sublayer: with layer dropping (``death_rate``) every sub-layer tosses its own coin instead of the layer
    # as a whole (reference: onmt/models/multilingual_translator/relative_transformer_layers.py:136-176)
    stochastic_sublayer = False

    def _survives(self, sublayer: bool = False) -> bool:
        """Coin of the layer (``sublayer`` False) or of one sub-layer; always True outside training / without dropping,
        and for sub-layers when the layer as a whole has already tossed."""
        if sublayer and not self.stochastic_sublayer:
            return True
        if not self.training or self.death_rate <= 0:
            return True
        return torch.rand(1).item() >= self.death_rate

    def _block(self, idx, norm, fn, x, p, seqs, *args, scale=None):
        """One residual sub-layer under the layer's structure switches; ``idx`` picks the rezero gate."""
        if self.rezero:
            g = self.gates[idx] if scale is None else self.gates[idx] * scale
            return _scaled_sub(self, fn, x, x, p, seqs, *args, scale=g)
        if self.post_norm:
            y = _sub(self, fn, x, x, p, seqs, *args) if scale is None else _scaled_sub(self, fn, x, x, p, seqs, *args, scale=scale)
            return norm(y)
        x, h = norm.with_residual(x)
        if scale is None:
            return _sub(self, fn, h, x, p, seqs, *args)
        return _scaled_sub(self, fn, h, x, p, seqs, *args, scale=scale)


class PackedConvolution(nn.Module):
    """Conformer convolution module on packed sequences: pointwise conv + GLU, depthwise conv over time (padding frames
    zeroed so that no sequence sees its neighbour or its padding), per-frame LayerNorm over the channels (a batch of one
    sequence and a padded batch give the same frames), SiLU, pointwise conv; called like the other
    sub-layers (``residual`` / ``dropout_p`` keywords)."""

    def __init__(self, dim: int, kernel: int = 31):
        super().__init__()
        if kernel % 2 == 0:
            raise ValueError("-conv_kernel must be odd (got %d)" % kernel)
        self.pw1 = nn.Conv1d(dim, 2 * dim, 1)
        self.dw = nn.Conv1d(dim, dim, kernel, padding=kernel // 2, groups=dim)
        self.norm = nn.LayerNorm(dim)
        self.pw2 = nn.Conv1d(dim, dim, 1)

    def forward(self, x, seqs: PackedSeqs, residual=None, dropout_p: float = 0.0):
        from ..ops.reference import unpad_packed
        padded = seqs.pad(x, time_first=False).float()                            # [B, T, C]
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
        valid = (torch.arange(padded.shape[1], device=x.device)[None, :] < lengths[:, None]).to(padded.dtype)
        h = F.glu(self.pw1((padded * valid.unsqueeze(-1)).transpose(1, 2)), dim=1) * valid.unsqueeze(1)
        h = F.silu(self.norm(self.dw(h).transpose(1, 2)))                          # [B, T, C]
        h = self.pw2(h.transpose(1, 2)).transpose(1, 2)
        y = unpad_packed(h.to(x.dtype), seqs.cu, x.shape[0])
        y = F.dropout(y, dropout_p, self.training) if dropout_p > 0 else y
        return y if residual is None else residual + y


def _over_time(seqs: PackedSeqs, x, fn):
    """Runs ``fn`` on the padded ``[B, C, T]`` view of packed rows ``x [N, C]`` (padding frames zero) and packs the result."""
    from ..ops.reference import unpad_packed
    padded = seqs.pad(x, time_first=False).float()
    lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
    valid = (torch.arange(padded.shape[1], device=x.device)[None, :] < lengths[:, None]).to(padded.dtype)
    y = fn((padded * valid.unsqueeze(-1)).transpose(1, 2)).transpose(1, 2)
    return unpad_packed(y.to(x.dtype).contiguous(), seqs.cu, x.shape[0])


class ConvolutionalGatingMLP(nn.Module):
    """cgMLP branch of a Branchformer layer: Linear(d -> u) + GELU, split into halves (r, g), ``r * GELU(dwconv(LN(g)))``,
    Linear(u/2 -> d).  The gate's convolution starts near zero with bias one, so the unit starts close to the identity
    on ``r``.  (reference: onmt/models/speech_recognizer/fairseq_wav2vec2/cgmlp.py:14-117)"""

    def __init__(self, dim: int, units: int, kernel: int = 31):
        super().__init__()
        self.proj1 = nn.Linear(dim, units)
        self.gate_norm = nn.LayerNorm(units // 2)
        self.gate_conv = nn.Conv1d(units // 2, units // 2, kernel, padding=(kernel - 1) // 2, groups=units // 2)
        nn.init.normal_(self.gate_conv.weight, std=1e-6)
        nn.init.ones_(self.gate_conv.bias)
        self.proj2 = nn.Linear(units // 2, dim)

    def forward(self, x, seqs: PackedSeqs):
        r, g = F.gelu(self.proj1(x.float())).chunk(2, dim=-1)
        g = _over_time(seqs, self.gate_norm(g), self.gate_conv)
        return self.proj2(r * F.gelu(g)).to(x.dtype)


class EncoderLayer(nn.Module, _LayerOptions):
    """Self-attention + FFN block.  Pre-LN: x += D(Attn(LN(x))); x += D(FFN(LN(x))).  Post-LN (``post_norm``):
    x = LN(x + D(Attn(x))); x = LN(x + D(FFN(x))).  Optional stochastic depth (``death_rate``), ``rezero``, ``macaron``
    and gated feed-forward (``glu``)."""

    def __init__(self, dim, heads, inner, dropout=0.1, attn_dropout=0.1, activation="relu", attn_bias=False,
                 death_rate=0.0, ffn_dropout=None, post_norm=False, rezero=False, macaron=False, glu=False):
        super().__init__()
        fd = dropout if ffn_dropout is None else ffn_dropout
        self.attn_norm = LayerNorm(dim)
        self.attn = SelfAttention(dim, heads, attn_dropout, bias=attn_bias)
        self.ffn_norm = LayerNorm(dim)
        self.ffn = FeedForward(dim, inner, fd, activation, glu=glu)
        self.dropout = dropout
        self.death_rate = death_rate
        self.conv = None
        self._init_options(dim, inner, fd, activation, post_norm, rezero, macaron, glu)

    def drop_ffn(self):
        """``-no_ffn``: the layer is attention (and the convolution block, if any) only.
        (reference: onmt/models/speech_recognizer/relative_transformer_layers.py:49, 89-96)"""
        self.ffn = self.ffn_norm = None

    def add_depthwise_conv(self, kernel: int = 31):
        """``-depthwise_conv``: a Conformer convolution block (pointwise GLU, depthwise convolution of ``kernel`` taps,
        normalisation, SiLU, pointwise) between the attention and the feed-forward block, with its own LayerNorm and
        residual.  (reference: onmt/models/speech_recognizer/relative_transformer_layers.py:136-143, 209-222)"""
        dim = self.attn_norm.weight.shape[0]
        self.conv_norm = LayerNorm(dim)
        self.conv = PackedConvolution(dim, kernel)

    def add_branchformer(self, cgmlp_kernel: int = 31, merge_kernel: int = 3):
        """``-branchformer``: next to the attention branch a cgMLP branch reads the same layer input; the two outputs are
        concatenated, a depthwise convolution over time is added to the concatenation, and a linear layer merges them
        into the residual.  The feed-forward block follows unchanged.  Pre-LayerNorm layers only.
        (reference: onmt/models/speech_recognizer/fairseq_wav2vec2/wav2vec2.py:1226-1246, 1504-1566)"""
        if self.post_norm or self.rezero:
            raise NotImplementedError("-branchformer is built for pre-LayerNorm layers")
        dim = self.attn_norm.weight.shape[0]
        self.cgmlp_norm = LayerNorm(dim)
        self.cgmlp = ConvolutionalGatingMLP(dim, 2 * dim, cgmlp_kernel)
        self.merge_conv = nn.Conv1d(2 * dim, 2 * dim, merge_kernel, padding=(merge_kernel - 1) // 2, groups=2 * dim)
        self.merge_proj = nn.Linear(2 * dim, dim)

    def _branchformer_block(self, x, seqs: PackedSeqs, p: float):
        a = self.attn(self.attn_norm(x), seqs, residual=None, dropout_p=p)
        c = F.dropout(self.cgmlp(self.cgmlp_norm(x), seqs), p, self.training)
        both = torch.cat([a, c], -1)
        merged = self.merge_proj((both + _over_time(seqs, both, self.merge_conv)).float())
        return x + F.dropout(merged, p, self.training).to(x.dtype)

    def forward(self, x, seqs: PackedSeqs):
        keep = self._survives
        if not self.stochastic_sublayer and not keep():
            return x
        p = self.dropout
        if self.macaron and keep(True):
            x = self._block(2, self.mcr_norm, self.mcr_ffn, x, p, seqs, scale=0.5)
        if getattr(self, "cgmlp", None) is not None:
            x = self._branchformer_block(x, seqs, p)
        elif keep(True):
            x = self._block(0, self.attn_norm, self.attn, x, p, seqs, seqs)
        if self.conv is not None and keep(True):
            x = self._block(4, self.conv_norm, self.conv, x, p, seqs, seqs)
        if self.ffn is not None and keep(True):
            x = self._block(1, self.ffn_norm, self.ffn, x, p, seqs, scale=self.ffn_scale)
        return x


class DecoderLayer(nn.Module, _LayerOptions):
    """Causal self-attention, encoder-decoder attention and FFN (pre- or post-LN).  ``interleaved_ffn`` adds a
    second FFN between the two attentions (the DeltaLM decoder layout); ``rezero`` / ``macaron`` / ``glu`` as in the
    encoder layer."""

    def __init__(self, dim, heads, inner, dropout=0.1, attn_dropout=0.1, activation="relu", attn_bias=False,
                 death_rate=0.0, ffn_dropout=None, ignore_source=False, post_norm=False, interleaved_ffn=False,
                 kv_dim=None, rezero=False, macaron=False, glu=False):
        super().__init__()
        fd = dropout if ffn_dropout is None else ffn_dropout
        self.self_norm = LayerNorm(dim)
        self.self_attn = SelfAttention(dim, heads, attn_dropout, bias=attn_bias, causal=True)
        self.ignore_source = ignore_source
        if interleaved_ffn:
            self.mid_norm = LayerNorm(dim)
            self.mid_ffn = FeedForward(dim, inner, fd, activation, glu=glu)
        self.interleaved_ffn = interleaved_ffn
        if not ignore_source:
            self.cross_norm = LayerNorm(dim)
            self.cross_attn = CrossAttention(dim, heads, attn_dropout, bias=attn_bias, kv_dim=kv_dim)
        self.ffn_norm = LayerNorm(dim)
        self.ffn = FeedForward(dim, inner, fd, activation, glu=glu)
        self.dropout = dropout
        self.death_rate = death_rate
        self._init_options(dim, inner, fd, activation, post_norm, rezero, macaron, glu)

    def forward(self, x, seqs: PackedSeqs, memory, mem_seqs: PackedSeqs):
        keep = self._survives
        if not self.stochastic_sublayer and not keep():
            return x
        p = self.dropout
        if self.macaron and keep(True):
            x = self._block(2, self.mcr_norm, self.mcr_ffn, x, p, seqs, scale=0.5)
        if keep(True):
            x = self._block(0, self.self_norm, self.self_attn, x, p, seqs, seqs)
        if self.interleaved_ffn and keep(True):
            x = self._block(4, self.mid_norm, self.mid_ffn, x, p, seqs)
        if not self.ignore_source and keep(True):
            x = self._block(3, self.cross_norm, self.cross_attn, x, p, seqs, seqs, memory, mem_seqs)
        if keep(True):
            x = self._block(1, self.ffn_norm, self.ffn, x, p, seqs, scale=self.ffn_scale)
        return x

    def step(self, x, cache: dict, mem_mask):
        if self.rezero or self.macaron:
            return self._step_general(x, cache, mem_mask)
        if self.post_norm:
            x = self.self_norm(x + self.self_attn.step(x, cache))
            if self.interleaved_ffn:
                x = self.mid_norm(self.mid_ffn(x, residual=x))
            if not self.ignore_source:
                x = self.cross_norm(x + self.cross_attn.step(x, cache, mem_mask))
            return self.ffn_norm(self.ffn(x, residual=x))
        x = self.self_attn.step(self.self_norm(x), cache, residual=x)      # residual add in the GEMM epilogue
        if self.interleaved_ffn:
            x = self.mid_ffn(self.mid_norm(x), residual=x)
        if not self.ignore_source:
            x = self.cross_attn.step(self.cross_norm(x), cache, mem_mask, residual=x)
        return self.ffn(self.ffn_norm(x), residual=x)


def _decoder_step_general(self, x, cache: dict, mem_mask):
    """Incremental step for the structure switches that the fast paths above do not cover (rezero gates, macaron)."""
    def blk(idx, norm, fn, x, scale=None):
        if self.rezero:
            g = self.gates[idx] if scale is None else self.gates[idx] * scale
            return x + (fn(x).float() * g).to(x.dtype)
        if self.post_norm:
            y = fn(x)
            return norm(x + (y if scale is None else (y.float() * scale).to(y.dtype)))
        y = fn(norm(x))
        return x + (y if scale is None else (y.float() * scale).to(y.dtype))
    if self.macaron:
        x = blk(2, self.mcr_norm, lambda h: self.mcr_ffn(h), x, 0.5)
    x = blk(0, self.self_norm, lambda h: self.self_attn.step(h, cache), x)
    if self.interleaved_ffn:
        x = blk(4, self.mid_norm, lambda h: self.mid_ffn(h), x)
    if not self.ignore_source:
        x = blk(3, self.cross_norm, lambda h: self.cross_attn.step(h, cache, mem_mask), x)
    return blk(1, self.ffn_norm, lambda h: self.ffn(h), x, self.ffn_scale)


DecoderLayer._step_general = _decoder_step_general


def pack_padded(x_bt, lengths, capacity=None):
    """Right-padded ``[B, T, ...]`` + lengths -> packed ``[N, ...]`` and a ``PackedSeqs`` descriptor (tokens unused)."""
    B, T = x_bt.shape[0], x_bt.shape[1]
    lengths = lengths.to(torch.int64).clamp(max=T)
    ar = torch.arange(T, device=x_bt.device)
    mask = ar[None, :] < lengths[:, None]
    packed = x_bt[mask]
    total = packed.shape[0]
    cap = capacity if capacity is not None else total
    if cap > total:
        packed = torch.cat([packed, packed.new_zeros((cap - total,) + tuple(packed.shape[1:]))], 0)
    cu = torch.zeros(B + 1, dtype=torch.int32, device=x_bt.device)
    cu[1:] = torch.cumsum(lengths, 0).to(torch.int32)
    pos = ar[None, :].expand(B, T)[mask]
    if cap > total:
        pos = torch.cat([pos, pos.new_zeros(cap - total)])
    seqs = PackedSeqs(torch.ones(cap, dtype=torch.int64, device=x_bt.device), pos, cu, int(T), lengths)
    return packed, seqs
