"""w2v-BERT 2.0 / Conformer-Shaw speech encoder family.

Pieces (reference: onmt/models/speech_recognizer/w2v_bert/): named size presets (config.py:160-255 ``_encoder_600m`` /
``_encoder_300m``, :283-330 ``600m`` pre-training arch), the filterbank front end that stacks ``fbank_stride`` frames
(w2vbert_feature_extractor.py, frontend.py), the span masker with a learned mask vector (masker.py), the Gumbel-softmax
product quantiser (vector_quantizer.py), the Conformer block with Shaw relative-position keys and a causal depthwise
convolution (w2vbert_conformer_shaw.py:29-82), and the two-loss pre-training model (w2vbert_wav2vec.py: contrastive loss
on the first N-K layers' output, masked-prediction cross-entropy over code-book ids on the last K layers).

FFN halves, projections and LayerNorms run on packed ``[frames, dim]`` matrices through the fused GEMM / LayerNorm
kernels; the attention scores carry an additive, query-dependent position term (``q . r[clip(j - i)]``), which the packed
tensor-core attention kernels do not take, so that sub-layer pads to ``[B, heads, T, T]`` and uses PyTorch's attention.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import FeedForward, LayerNorm, Linear, PackedSeqs, SelfAttention, pack_padded
from .speech_encoders import compute_mask_spans, split_audio_batch


@dataclass
class ConformerShawConfig:
    model_dim: int = 1024
    feature_dim: int = 160            # num_fbank_channels * fbank_stride
    num_fbank_channels: int = 80
    fbank_stride: int = 2
    layers: int = 24
    heads: int = 16
    ffn_dim: int = 4096
    dropout: float = 0.0
    attn_dropout: float = 0.0
    layer_drop: float = 0.0
    conv_kernel: int = 31
    causal_conv: bool = True
    max_left: int = 64                # Shaw clipping window
    max_right: int = 8
    max_seq_len: int = 4096


@dataclass
class W2VBertConfig:
    encoder: ConformerShawConfig = field(default_factory=ConformerShawConfig)
    final_dim: int = 768
    temporal_mask_span: int = 10
    max_temporal_mask_prob: float = 0.65
    quantized_dim: int = 1024
    num_codebooks: int = 1
    num_codebook_entries: int = 1024
    codebook_temperature: Tuple[float, float, float] = (2.0, 0.1, 0.999995)
    num_distractors: int = 100
    logit_temp: float = 0.1
    diversity_loss_weight: float = 0.2
    num_bert_layers: int = 16
    num_target_codebooks: int = 1
    w2v2_loss_weight: float = 1.0
    bert_loss_weight: float = 1.0
    bert_label_smoothing: float = 0.0


def w2vbert_arch(name: str) -> W2VBertConfig:
    """Presets by name: ``600m`` (24 layers), ``300m`` (12 layers), ``test`` (tiny, for unit tests)."""
    name = name.lower()
    if name in ("600m", "w2v-bert-2.0", "w2vbert"):
        return W2VBertConfig()
    if name == "300m":
        return W2VBertConfig(encoder=ConformerShawConfig(layers=12), num_bert_layers=8)
    if name == "test":
        enc = ConformerShawConfig(model_dim=64, layers=3, heads=4, ffn_dim=128, conv_kernel=7, max_left=8, max_right=2)
        return W2VBertConfig(encoder=enc, final_dim=32, quantized_dim=32, num_codebooks=2, num_codebook_entries=16,
                             num_distractors=5, num_bert_layers=1, num_target_codebooks=2)
    raise ValueError("unknown w2v-BERT architecture %r" % name)


class FbankFrontend(nn.Module):
    """``[B, T, 80]`` log-mel frames -> ``[B, T // stride, stride * 80]`` stacked frames -> LayerNorm -> model dim."""

    def __init__(self, cfg: ConformerShawConfig):
        super().__init__()
        self.stride, self.channels = cfg.fbank_stride, cfg.num_fbank_channels
        self.norm = nn.LayerNorm(cfg.feature_dim)
        self.proj = nn.Linear(cfg.feature_dim, cfg.model_dim)

    def extract(self, feats, lengths):
        B, T, C = feats.shape
        if C == self.channels * self.stride:        # frames were stacked by the data pipeline already
            return self.norm(feats.float()), lengths
        T2 = T // self.stride
        stacked = feats[:, :T2 * self.stride].reshape(B, T2, C * self.stride)
        return self.norm(stacked.float()), torch.div(lengths, self.stride, rounding_mode="floor").clamp(min=1, max=max(T2, 1))

    def forward(self, feats, lengths):
        x, lengths = self.extract(feats, lengths)
        return self.proj(x), x, lengths


class SpanMasker(nn.Module):
    """Replaces random spans of frames with one learned vector; returns the boolean ``[B, T]`` mask it drew."""

    def __init__(self, dim: int, span: int, max_prob: float):
        super().__init__()
        self.span, self.max_prob = span, max_prob
        self.mask_vector = nn.Parameter(torch.empty(dim).uniform_())

    def forward(self, x, lengths, generator=None):
        B, T, _ = x.shape
        mask = compute_mask_spans(B, T, lengths, self.max_prob, self.span, generator).to(x.device)
        mask = mask & (torch.arange(T, device=x.device)[None, :] < lengths[:, None])
        return torch.where(mask.unsqueeze(-1), self.mask_vector.to(x.dtype), x), mask


class GumbelVectorQuantizer(nn.Module):
    """Product quantiser: ``G`` code books of ``V`` entries of ``quantized_dim / G`` values; training draws entries with
    the straight-through Gumbel softmax at a temperature that decays per update, evaluation takes the arg-max."""

    def __init__(self, in_dim: int, out_dim: int, groups: int, entries: int, temperature=(2.0, 0.5, 0.999995)):
        super().__init__()
        assert out_dim % groups == 0
        self.groups, self.entries = groups, entries
        self.t_max, self.t_min, self.t_decay = temperature
        self.updates = 0
        self.logits = nn.Linear(in_dim, groups * entries)
        nn.init.normal_(self.logits.weight, 0.0, 1.0)
        nn.init.zeros_(self.logits.bias)
        self.codebook = nn.Parameter(torch.empty(groups, entries, out_dim // groups).uniform_())

    @property
    def temperature(self) -> float:
        return max(self.t_max * self.t_decay ** self.updates, self.t_min)

    def forward(self, x):
        """x ``[N, in_dim]`` -> (quantised ``[N, out_dim]``, code ids ``[N, G]``, diversity loss, code perplexity)."""
        N = x.shape[0]
        logits = self.logits(x.float()).view(N, self.groups, self.entries)
        ids = logits.argmax(-1)
        hard = F.one_hot(ids, self.entries).float()
        usage = hard.mean(0)
        code_ppl = torch.exp(-(usage * torch.log(usage + 1e-7)).sum(-1)).sum()
        soft = logits.softmax(-1).mean(0)
        prob_ppl = torch.exp(-(soft * torch.log(soft + 1e-7)).sum(-1)).sum()
        if self.training:
            onehot = F.gumbel_softmax(logits, tau=self.temperature, hard=True, dim=-1)
            self.updates += 1
        else:
            onehot = hard
        q = torch.einsum("ngv,gvd->ngd", onehot, self.codebook).reshape(N, -1)
        total = self.groups * self.entries
        return q, ids, (total - prob_ppl) / total, code_ppl


class ShawRelPosSelfAttention(SelfAttention):
    """Self-attention whose scores get ``q_i . r[clip(j - i, -max_left, max_right)]`` added (Shaw et al. relative keys).

    The term is computed as one ``[.., T, L+R+1]`` product against the small table and gathered to ``[T, T]``, so its
    cost is independent of the sequence length squared times the head size."""

    def __init__(self, dim, heads, attn_dropout=0.0, max_left=64, max_right=8):
        super().__init__(dim, heads, attn_dropout, bias=True)
        self.max_left, self.max_right = max_left, max_right
        self.rel_k = nn.Embedding(max_left + max_right + 1, dim // heads)
        nn.init.xavier_uniform_(self.rel_k.weight)

    def rel_index(self, T: int, device):
        pos = torch.arange(T, device=device)
        return (pos[None, :] - pos[:, None]).clamp(-self.max_left, self.max_right) + self.max_left     # [T, T]

    def forward(self, x, seqs: PackedSeqs, residual=None, dropout_p: float = 0.0):
        from ..ops.reference import pad_packed
        H, h = self.dim, self.heads
        qkv = self.qkv(x)                                                              # packed [N, 3H]
        T = int(seqs.max_len)
        scale = (H // h) ** -0.5
        q_rows = qkv[:, :H].float().view(-1, h, H // h)
        by_offset = torch.matmul(q_rows, self.rel_k.weight.float().t()) * scale         # [N, h, L+R+1]
        by_offset, _ = pad_packed(by_offset.reshape(by_offset.shape[0], -1), seqs.cu, T)    # [B, T, h * (L+R+1)]
        B = by_offset.shape[0]
        by_offset = by_offset.view(B, T, h, -1).transpose(1, 2)                         # [B, h, T, L+R+1]
        bias = by_offset.gather(-1, self.rel_index(T, x.device)[None, None].expand(B, h, T, T))
        # the relative-key term is an additive operand of the attention kernels (gradient comes back in the same layout)
        ctx = ops.self_attention(qkv, seqs.cu, h, T, False, self.attn_dropout, self.training, scale=scale, bias=bias)
        return self.out(ctx.to(x.dtype), dropout_p=dropout_p, residual=residual)


class ShawConvolution(nn.Module):
    """Point-wise conv + GLU -> depthwise conv (left-padded when causal) -> LayerNorm over channels -> SiLU -> point-wise."""

    def __init__(self, dim: int, kernel: int, causal: bool):
        super().__init__()
        self.kernel, self.causal = kernel, causal
        self.pw1 = nn.Conv1d(dim, 2 * dim, 1, bias=False)
        self.dw = nn.Conv1d(dim, dim, kernel, padding=0 if causal else kernel // 2, groups=dim, bias=False)
        self.norm = nn.LayerNorm(dim)
        self.pw2 = nn.Conv1d(dim, dim, 1, bias=False)

    def forward(self, x_bt, valid):                  # [B, T, C], valid [B, T] float
        x = (x_bt.float() * valid.unsqueeze(-1)).transpose(1, 2)
        x = F.glu(self.pw1(x), dim=1) * valid.unsqueeze(1)
        if self.causal:
            x = F.pad(x, (self.kernel - 1, 0))
        x = self.dw(x)
        x = F.silu(self.norm(x.transpose(1, 2))).transpose(1, 2)
        return self.pw2(x).transpose(1, 2)


class ConformerShawBlock(nn.Module):
    def __init__(self, cfg: ConformerShawConfig):
        super().__init__()
        d = cfg.model_dim
        self.ffn1_norm, self.ffn1 = LayerNorm(d), FeedForward(d, cfg.ffn_dim, cfg.dropout, "silu")
        self.attn_norm = LayerNorm(d)
        self.attn = ShawRelPosSelfAttention(d, cfg.heads, cfg.attn_dropout, cfg.max_left, cfg.max_right)
        self.conv_norm, self.conv = LayerNorm(d), ShawConvolution(d, cfg.conv_kernel, cfg.causal_conv)
        self.ffn2_norm, self.ffn2 = LayerNorm(d), FeedForward(d, cfg.ffn_dim, cfg.dropout, "silu")
        self.final_norm = LayerNorm(d)
        self.dropout = cfg.dropout

    def forward(self, x, seqs: PackedSeqs):
        from ..ops.reference import unpad_packed
        x = x + 0.5 * self.ffn1(self.ffn1_norm(x), dropout_p=self.dropout)
        x = self.attn(self.attn_norm(x), seqs, residual=x, dropout_p=self.dropout)
        padded = seqs.pad(self.conv_norm(x), time_first=False)
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
        valid = (torch.arange(padded.shape[1], device=x.device)[None, :] < lengths[:, None]).float()
        c = unpad_packed(self.conv(padded, valid).to(x.dtype), seqs.cu, x.shape[0])
        x = x + F.dropout(c, self.dropout, self.training)
        x = x + 0.5 * self.ffn2(self.ffn2_norm(x), dropout_p=self.dropout)
        return self.final_norm(x)


class ConformerShawEncoder(nn.Module):
    """Front end + Conformer-Shaw stack; ``forward(source)`` returns packed frames and their ``PackedSeqs`` like the other
    speech encoders, so it plugs into ``SpeechToTextModel`` (``-enc_pretrained_model w2vbert``)."""

    def __init__(self, cfg: Optional[ConformerShawConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or ConformerShawConfig()
        self.frontend = FbankFrontend(cfg)
        self.layers = nn.ModuleList([ConformerShawBlock(cfg) for _ in range(cfg.layers)])
        self.dim = cfg.model_dim

    def _fused(self) -> bool:
        return ops.fused_param(self.layers[0].final_norm.weight)

    def run_layers(self, packed, seqs, first: int = 0, last: Optional[int] = None):
        for layer in self.layers[first:last]:
            if self.training and self.cfg.layer_drop > 0 and torch.rand(()).item() < self.cfg.layer_drop:
                continue
            packed = layer(packed, seqs)
        return packed

    def embed(self, source):
        feats, lengths = split_audio_batch(source)
        x, raw, lengths = self.frontend(feats, lengths.to(feats.device))
        return x, raw, lengths

    def forward(self, source):
        x, _, lengths = self.embed(source)
        x = F.dropout(x, self.cfg.dropout, self.training)
        packed, seqs = pack_padded(x, lengths)
        if packed.is_cuda and self._fused():
            packed = packed.to(torch.bfloat16)
        return self.run_layers(packed, seqs), seqs


class W2VBertModel(nn.Module):
    """Pre-training model: masked frames go through the first ``N - K`` blocks, whose output is scored against the
    quantised unmasked features with a contrastive loss (true code vs sampled distractors of the same utterance); the
    last ``K`` blocks continue and predict the code-book ids of the masked frames with cross-entropy."""

    def __init__(self, cfg: Optional[W2VBertConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or W2VBertConfig()
        e = cfg.encoder
        assert 0 < cfg.num_bert_layers < e.layers and cfg.num_target_codebooks <= cfg.num_codebooks
        self.encoder = ConformerShawEncoder(e)
        self.masker = SpanMasker(e.model_dim, cfg.temporal_mask_span, cfg.max_temporal_mask_prob)
        self.quantizer = GumbelVectorQuantizer(e.feature_dim, cfg.quantized_dim, cfg.num_codebooks,
                                               cfg.num_codebook_entries, cfg.codebook_temperature)
        self.final_proj = nn.Linear(e.model_dim, cfg.final_dim)
        self.final_target_proj = nn.Linear(cfg.quantized_dim, cfg.final_dim)
        self.bert_proj = nn.Linear(e.model_dim, cfg.num_codebook_entries * cfg.num_target_codebooks)

    def _distractors(self, targets, batch_of, generator=None):
        """For every masked frame, ``num_distractors`` other masked frames of the same utterance: ``[M, D, dim]``."""
        M, D = targets.shape[0], self.cfg.num_distractors
        counts = torch.bincount(batch_of, minlength=int(batch_of.max()) + 1 if M else 1)
        first = torch.cumsum(counts, 0) - counts
        n = counts[batch_of].clamp(min=2)                                  # frames masked in my utterance
        mine = torch.arange(M, device=targets.device) - first[batch_of]
        draw = (torch.rand(M, D, generator=generator).to(targets.device) * (n - 1)[:, None]).long()
        draw = draw + (draw >= mine[:, None]).long()                       # skip myself
        idx = (first[batch_of][:, None] + draw).clamp(max=M - 1)
        return targets[idx]

    def forward(self, source, generator=None):
        cfg, enc = self.cfg, self.encoder
        x, raw, lengths = enc.embed(source)
        x, mask = self.masker(F.dropout(x, enc.cfg.dropout, self.training), lengths, generator)
        packed, seqs = pack_padded(x, lengths)
        valid = torch.arange(x.shape[1], device=x.device)[None, :] < lengths[:, None]
        flat_mask = mask[valid]                                            # masked frames among the packed rows
        batch_of = torch.arange(x.shape[0], device=x.device)[:, None].expand_as(valid)[valid][flat_mask]
        if packed.is_cuda and enc._fused():
            packed = packed.to(torch.bfloat16)
        split = len(enc.layers) - cfg.num_bert_layers
        mid = enc.run_layers(packed, seqs, 0, split)
        out = enc.run_layers(mid, seqs, split, None)

        q, ids, diversity, code_ppl = self.quantizer(raw[valid][flat_mask])
        tgt = self.final_target_proj(q)
        pred = self.final_proj(mid[:flat_mask.shape[0]][flat_mask].float())
        cand = torch.cat([tgt.unsqueeze(1), self._distractors(tgt, batch_of, generator)], 1)     # [M, 1 + D, dim]
        sim = F.cosine_similarity(pred.unsqueeze(1), cand, dim=-1) / cfg.logit_temp
        same = (cand[:, 1:] == tgt.unsqueeze(1)).all(-1)                   # a distractor equal to the target is no negative
        sim = torch.cat([sim[:, :1], sim[:, 1:].masked_fill(same, float("-inf"))], 1)
        contrastive = F.cross_entropy(sim, torch.zeros(sim.shape[0], dtype=torch.long, device=sim.device), reduction="sum")
        w2v2_loss = contrastive + cfg.diversity_loss_weight * diversity * sim.shape[0]

        logits = self.bert_proj(out[:flat_mask.shape[0]][flat_mask].float())
        logits = logits.view(-1, cfg.num_target_codebooks, cfg.num_codebook_entries)
        bert_loss = F.cross_entropy(logits.reshape(-1, cfg.num_codebook_entries), ids[:, :cfg.num_target_codebooks].reshape(-1),
                                    reduction="sum", label_smoothing=cfg.bert_label_smoothing)
        loss = cfg.w2v2_loss_weight * w2v2_loss + cfg.bert_loss_weight * bert_loss
        return {"loss": loss, "w2v2_loss": w2v2_loss.detach(), "bert_loss": bert_loss.detach(), "contrastive": contrastive.detach(),
                "diversity": diversity.detach(), "code_perplexity": code_ppl.detach(), "num_masked": int(flat_mask.sum()),
                "bert_accuracy": (logits.argmax(-1) == ids[:, :cfg.num_target_codebooks]).float().mean().detach()}


def build_w2vbert_encoder(opt, cfg_json: Optional[dict] = None) -> ConformerShawEncoder:
    """Encoder for ``-enc_pretrained_model w2vbert*`` / ``xeus``.  A name that carries ``600m`` or ``300m`` selects that
    preset; any other name builds the architecture at the sizes of the command line (``-model_size``, ``-encoder_layers``
    or ``-layers``, ``-n_heads``, ``-inner_size``, ``-input_size`` filterbank channels).  Keys of an ``-enc_config_file``
    JSON (``model_dim``, ``num_encoder_layers``, ...) and the dropout flags override either."""
    name = (getattr(opt, "enc_pretrained_model", "") or "").lower()
    if "600m" in name or "300m" in name:
        cfg = w2vbert_arch("300m" if "300m" in name else "600m").encoder
    else:
        n_layers = getattr(opt, "encoder_layers", -1)
        cfg = ConformerShawConfig(model_dim=opt.model_size, layers=n_layers if n_layers and n_layers > 0 else opt.layers,
                                  heads=opt.n_heads, ffn_dim=opt.inner_size,
                                  num_fbank_channels=int(getattr(opt, "input_size", 80) or 80),
                                  conv_kernel=int(getattr(opt, "conv_kernel", 31) or 31))
    j = cfg_json or {}
    for key, attr in (("model_dim", "model_dim"), ("num_encoder_layers", "layers"), ("num_encoder_attn_heads", "heads"),
                      ("ffn_inner_dim", "ffn_dim"), ("depthwise_conv_kernel_size", "conv_kernel"),
                      ("num_fbank_channels", "num_fbank_channels"), ("fbank_stride", "fbank_stride")):
        if key in j:
            setattr(cfg, attr, int(j[key]))
    cfg.feature_dim = cfg.num_fbank_channels * cfg.fbank_stride
    cfg.dropout = float(getattr(opt, "enc_pretrain_hidden_dropout", getattr(opt, "dropout", 0.0)) or 0.0)
    cfg.attn_dropout = float(getattr(opt, "attn_dropout", 0.0) or 0.0)
    cfg.layer_drop = float(getattr(opt, "death_rate", 0.0) or 0.0) / 2
    return ConformerShawEncoder(cfg)
