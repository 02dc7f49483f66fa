"""Model families built around pretrained-style encoders / decoders, all on the packed fused layers:

* ``PretrainedStyleDecoder`` - mBART / mBART-50 / BART / M2M-100 / Whisper / DeltaLM decoders as one configurable stack
  (learned or sinusoidal positions with offset, embedding LayerNorm, pre- or post-LN, GELU/ReLU, biases, optional
  interleaved FFN for DeltaLM, tied output projection);
* ``PretrainedStyleEncoder`` - the matching text encoders (mBART / BART / M2M-100 / DeltaLM);
* composite models registered under the reference's names: ``wav2vec2_bert`` (speech encoder + pretrained-style
  decoder, optional CTC head), ``wav2vec2_transformer``, ``whisper``, ``speech_transformer``,
  ``pretrain_transformer`` (text encoder + decoder of a chosen family), ``deltalm``.

Sizes come from the reference's json configs when given (``-enc_config_file`` / ``-dec_config_file``, Hugging Face style
keys), else from the training options.  Reference: pretrain_module/modeling_mbart.py:1598-2276 (encoder, decoder,
``step``), onmt/models/deltalm/transformer_decoder.py:21-423, onmt/models/whisper/whisper_decoder.py:341-827,
onmt/models/speech_recognizer/wav2vec2.py:522-1376 (``Wav2vecTransformer``, ``Wav2vecBERT``),
onmt/model_factory.py:146-731.
"""
from __future__ import annotations

import json
import math
from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import DecoderLayer, Embedding, EncoderLayer, LayerNorm, PackedSeqs
from .speech_encoders import SpeechTransformerEncoder, Wav2Vec2Encoder, WhisperEncoder
from .transformer import DecodingState, Generator, Seq2SeqBase, single_language

FAMILY_DEFAULTS = {
    # learned positions, position offset, embedding LayerNorm, final LayerNorm, pre-LN, scale embeddings, activation
    "mbart": dict(learned_pos=True, pos_offset=2, emb_norm=True, final_norm=True, pre_norm=True, scale=True, act="gelu"),
    "mbart50": dict(learned_pos=True, pos_offset=2, emb_norm=True, final_norm=True, pre_norm=True, scale=True, act="gelu"),
    "bart": dict(learned_pos=True, pos_offset=2, emb_norm=True, final_norm=False, pre_norm=False, scale=False, act="gelu"),
    "m2m100": dict(learned_pos=False, pos_offset=2, emb_norm=False, final_norm=True, pre_norm=True, scale=True, act="relu"),
    "m2m": dict(learned_pos=False, pos_offset=2, emb_norm=False, final_norm=True, pre_norm=True, scale=True, act="relu"),
    "deltalm": dict(learned_pos=True, pos_offset=2, emb_norm=True, final_norm=False, pre_norm=False, scale=True, act="gelu",
                    interleaved=True),
    "whisper": dict(learned_pos=True, pos_offset=0, emb_norm=False, final_norm=True, pre_norm=True, scale=False, act="gelu"),
    "bert": dict(learned_pos=True, pos_offset=0, emb_norm=True, final_norm=False, pre_norm=False, scale=False, act="gelu"),
    "roberta": dict(learned_pos=True, pos_offset=2, emb_norm=True, final_norm=False, pre_norm=False, scale=False, act="gelu"),
}


def load_json_config(path: Optional[str]) -> SimpleNamespace:
    if not path:
        return SimpleNamespace()
    with open(path) as fh:
        return SimpleNamespace(**json.load(fh))


def _cfg(cfg, names, default):
    for n in names:
        if hasattr(cfg, n):
            return getattr(cfg, n)
    return default


class PretrainedStyleDecoder(nn.Module):
    def __init__(self, family: str, vocab: int, dim: int, layers: int, heads: int, ffn: int, dropout=0.1, attn_dropout=0.0,
                 max_positions=1024, pad_idx=1, layerdrop=0.0, kv_dim=None, emb_dropout=None, word_dropout=0.0):
        super().__init__()
        f = FAMILY_DEFAULTS[family]
        self.family = family
        self.emb_dropout = dropout if emb_dropout is None else emb_dropout
        self.embed = Embedding(vocab, dim, pad_idx, scale=math.sqrt(dim) if f["scale"] else 1.0, max_pos=max_positions,
                               learned_pos=f["learned_pos"], pos_offset=f["pos_offset"])
        self.emb_norm = LayerNorm(dim) if f["emb_norm"] else None
        self.layers = nn.ModuleList([
            DecoderLayer(dim, heads, ffn, dropout, attn_dropout, f["act"], attn_bias=True, death_rate=layerdrop,
                         post_norm=not f["pre_norm"], interleaved_ffn=f.get("interleaved", False), kv_dim=kv_dim)
            for _ in range(layers)])
        self.final_norm = LayerNorm(dim) if f["final_norm"] else None
        self.dropout = dropout
        self.embed.word_dropout = word_dropout
        self.adapters = None

    def add_adapters(self, n_languages: int, location: int = 1, downsample: int = 4):
        """``-decoder_adapter``: one bottleneck adapter per language behind every decoder layer (``x + adapter_lang(x)``
        after the feed-forward block), chosen by the batch's target language
        (reference: pretrain_module/modeling_mbart.py:1039-1051, 1277-1283, 1844-1847)."""
        from .multilingual import MultilingualAdapter
        if location != 1:
            raise NotImplementedError("-decoder_adapter %d: only location 1 (behind each layer) is built" % location)
        dim = self.embed.weight.shape[1]
        self.adapters = nn.ModuleList([MultilingualAdapter(dim, dim // downsample, n_languages) for _ in self.layers])

    def _embed(self, seqs: PackedSeqs):
        if self.emb_norm is None:
            return self.embed(seqs, self.emb_dropout)
        return ops.dropout_add(self.emb_norm(self.embed(seqs, 0.0)), None, self.emb_dropout, self.training)

    def forward(self, tgt: PackedSeqs, memory, src: PackedSeqs, lang: Optional[int] = None):
        if self.adapters is not None and lang is None:
            raise ValueError("this decoder has language adapters: the batch must carry its target language id")
        x = self._embed(tgt)
        for i, layer in enumerate(self.layers):
            x = layer(x, tgt, memory, src)
            if self.adapters is not None:
                x = self.adapters[i](x, lang)
        return self.final_norm(x) if self.final_norm is not None else x

    def step(self, tokens, position: int, state: DecodingState):
        B = tokens.shape[0]
        seqs = PackedSeqs(tokens, torch.full_like(tokens, position), torch.arange(B + 1, dtype=torch.int32, device=tokens.device), 1)
        x = self.embed(seqs, 0.0)
        if self.emb_norm is not None:
            x = self.emb_norm(x)
        for i, layer in enumerate(self.layers):
            x = layer.step(x, state.buffers[i], state.src_pad_mask)
            if self.adapters is not None:
                x = self.adapters[i](x, int(state.tgt_lang.view(-1)[0]))
        return self.final_norm(x) if self.final_norm is not None else x


class PretrainedStyleEncoder(nn.Module):
    def __init__(self, family: str, vocab: int, dim: int, layers: int, heads: int, ffn: int, dropout=0.1, attn_dropout=0.0,
                 max_positions=1024, pad_idx=1, layerdrop=0.0, embed: Optional[Embedding] = None):
        super().__init__()
        f = FAMILY_DEFAULTS[family]
        self.embed = embed or Embedding(vocab, dim, pad_idx, scale=math.sqrt(dim) if f["scale"] else 1.0,
                                        max_pos=max_positions, learned_pos=f["learned_pos"], pos_offset=f["pos_offset"])
        self.emb_norm = LayerNorm(dim) if f["emb_norm"] else None
        self.layers = nn.ModuleList([EncoderLayer(dim, heads, ffn, dropout, attn_dropout, f["act"], attn_bias=True,
                                                  death_rate=layerdrop, post_norm=not f["pre_norm"]) for _ in range(layers)])
        self.final_norm = LayerNorm(dim) if f["final_norm"] else None
        self.dropout = dropout

    def forward(self, src: PackedSeqs):
        x = self.embed(src, 0.0 if self.emb_norm is not None else self.dropout)
        if self.emb_norm is not None:
            x = ops.dropout_add(self.emb_norm(x), None, self.dropout, self.training)
        for layer in self.layers:
            x = layer(x, src)
        return self.final_norm(x) if self.final_norm is not None else x


def _decoder_family(opt) -> str:
    name = (getattr(opt, "dec_pretrained_model", "") or "").lower()
    for fam in ("mbart50", "mbart", "deltalm", "m2m100", "m2m", "bart", "roberta", "bert", "whisper"):
        if fam in name:
            return fam
    return "mbart50"


def _encoder_family(opt) -> str:
    name = (getattr(opt, "enc_pretrained_model", "") or "").lower()
    for fam in ("mbart50", "mbart", "deltalm", "m2m100", "m2m", "bart", "roberta", "bert"):
        if fam in name:
            return fam
    return "mbart50"


def build_pretrained_decoder(opt, vocab: int, family: Optional[str] = None, kv_dim=None) -> PretrainedStyleDecoder:
    fam = family or _decoder_family(opt)
    cfg = load_json_config(getattr(opt, "dec_config_file", ""))
    dim = _cfg(cfg, ["d_model", "decoder_embed_dim", "hidden_size"],
               opt.dec_pretrain_hidden_size if getattr(opt, "dec_pretrain_hidden_size", 768) != 768 else opt.model_size)
    return PretrainedStyleDecoder(
        fam, _cfg(cfg, ["vocab_size"], vocab), dim,
        _cfg(cfg, ["decoder_layers", "num_hidden_layers"], opt.layers),
        _cfg(cfg, ["decoder_attention_heads", "num_attention_heads"], opt.n_heads),
        _cfg(cfg, ["decoder_ffn_dim", "decoder_ffn_embed_dim", "intermediate_size"], opt.inner_size),
        # -dec_pretrain_hidden_dropout / -dec_pretrain_attn_dropout override the shared rates for a pretrained-style decoder
        # when they are moved off their defaults (reference: onmt/model_factory.py:636-644)
        dropout=opt.dec_pretrain_hidden_dropout if getattr(opt, "dec_pretrain_hidden_dropout", 0.1) != 0.1 else opt.dropout,
        attn_dropout=opt.dec_pretrain_attn_dropout if getattr(opt, "dec_pretrain_attn_dropout", 0.1) != 0.1 else opt.attn_dropout,
        emb_dropout=getattr(opt, "dec_pretrain_emb_dropout", 0.1) if getattr(opt, "dec_pretrain_emb_dropout", 0.1) != 0.1 else None,
        word_dropout=float(getattr(opt, "dec_pretrain_word_dropout", 0.0) or 0.0),
        max_positions=_cfg(cfg, ["max_position_embeddings", "max_target_positions"], 1024),
        pad_idx=_cfg(cfg, ["pad_token_id"], getattr(opt, "pad_idx", 1)), layerdrop=getattr(opt, "death_rate", 0.0), kv_dim=kv_dim)


def ctc_compress(context, seqs: PackedSeqs, logits, mode: str = "avg"):
    """Collapse consecutive frames of a sequence that share the CTC arg-max symbol into one state.

    ``mode``: ``avg`` (mean of the run), ``weighted`` (mean weighted by the probability of the predicted symbol) or
    ``softmax`` (weights = softmax of those probabilities within the run).  Returns the compressed packed states and
    their ``PackedSeqs`` (reference: onmt/models/speech_recognizer/ctc_compressor.py:11,
    onmt/models/speech_recognizer/wav2vec2.py:993-1017)."""
    N = context.shape[0]
    cu = seqs.cu.long()
    n_valid = int(cu[-1])
    pred = logits.argmax(-1)
    prob = torch.softmax(logits.float(), -1).gather(1, pred[:, None]).squeeze(1)
    idx = torch.arange(N, device=context.device)
    start = torch.ones(N, dtype=torch.bool, device=context.device)
    start[1:] = pred[1:] != pred[:-1]
    start[cu[:-1].clamp(max=N - 1)] = True                                  # a run never crosses a sentence boundary
    valid = idx < n_valid
    start &= valid
    seg = torch.cumsum(start.long(), 0) - 1                                 # run index of every frame
    n_seg = int(start.sum())
    seg = seg.clamp(min=0)
    if mode == "weighted":
        w = prob
    elif mode == "softmax":
        e = torch.exp(prob - prob.max())
        w = e
    else:
        w = torch.ones_like(prob)
    w = w * valid
    num = torch.zeros(n_seg, context.shape[1], dtype=torch.float32, device=context.device).index_add_(0, seg, context.float() * w[:, None])
    den = torch.zeros(n_seg, dtype=torch.float32, device=context.device).index_add_(0, seg, w)
    out = (num / den.clamp_min(1e-9)[:, None]).to(context.dtype)
    sent = torch.bucketize(idx, cu[1:].contiguous(), right=True).clamp(max=cu.numel() - 2)
    per_sent = torch.zeros(cu.numel() - 1, dtype=torch.long, device=context.device).index_add_(0, sent[start], torch.ones(n_seg, dtype=torch.long, device=context.device))
    new_cu = torch.zeros_like(seqs.cu)
    new_cu[1:] = torch.cumsum(per_sent, 0).to(seqs.cu.dtype)
    positions = torch.arange(n_seg, device=context.device) - new_cu.long()[:-1].repeat_interleave(per_sent)
    new_seqs = PackedSeqs(torch.zeros(n_seg, dtype=torch.long, device=context.device), positions, new_cu, int(per_sent.max()) if n_seg else 1)
    return out, new_seqs


class _ReferenceNaming:
    """Checkpoints of these families are written with the reference's parameter names and its fused-attention layout
    (``decoder.layers.3.self_attn.proj_weight`` ..., see ``pretrained_io``), and files written by the reference - or
    pretrained files in Hugging Face / fairseq naming - load back through the same maps."""

    def _io_parts(self):
        from . import pretrained_io as io
        enc, dec = self.encoder, self.decoder
        inter = any(getattr(l, "interleaved_ffn", False) for l in getattr(dec, "layers", []))
        speech = hasattr(enc, "extractor")
        # the reference keeps the fairseq model inside a wrapper module (onmt/models/speech_recognizer/wav2vec2.py:165)
        enc_prefix = "encoder.wav2vec_encoder." if speech else "encoder."
        return io, enc, dec, inter, speech, enc_prefix

    def to_reference_state_dict(self, sd):
        io, enc, dec, inter, speech, enc_prefix = self._io_parts()
        f32 = lambda t: t.detach().float().cpu().clone()
        sd = {k: f32(v) for k, v in sd.items()}
        e = {k[len("encoder."):]: v for k, v in sd.items() if k.startswith("encoder.")}
        d = {k[len("decoder."):]: v for k, v in sd.items() if k.startswith("decoder.")}
        out = {}
        if speech:
            conv = io.wav2vec2_to_reference(e, io._heads_of(enc), getattr(enc.extractor, "mode", "layer_norm") == "layer_norm")
        else:
            conv = io.text_encoder_to_reference(e, io._heads_of(enc))
        covered = set()
        for k, v in conv.items():
            out[enc_prefix + k] = v
        back = io.wav2vec2_to_native(conv, io._heads_of(enc)) if speech else (
            io.whisper_encoder_to_native(conv, io._heads_of(enc)) if hasattr(enc, "conv1") else io.text_encoder_to_native(conv, io._heads_of(enc)))
        covered.update("encoder." + k for k in back)
        dconv = io.decoder_to_reference(d, io._heads_of(dec), inter)
        for k, v in dconv.items():
            out["decoder." + k] = v
        covered.update("decoder." + k for k in io.decoder_to_native(dconv, io._heads_of(dec), inter))
        if "generator.weight" in sd:
            out["generator.0.linear.weight"] = sd["generator.weight"]
            covered.add("generator.weight")
        if "generator.bias" in sd:
            out["generator.0.linear.bias"] = sd["generator.bias"]
            covered.add("generator.bias")
        for k, v in sd.items():           # anything without a counterpart in the reference keeps its own name
            if k not in covered and k not in out:
                out[k] = v
        return out

    def from_reference_state_dict(self, ref_sd, target_keys=None):
        io, enc, dec, inter, speech, _ = self._io_parts()
        out = {}
        e = {k: v for k, v in ref_sd.items() if k.startswith("encoder.")}
        d = {k[len("decoder."):]: v for k, v in ref_sd.items() if k.startswith("decoder.")}
        if speech:
            e = {k[len("encoder."):]: v for k, v in e.items()}
            native = io.wav2vec2_to_native(e, io._heads_of(enc))
        elif hasattr(enc, "conv1"):
            native = io.whisper_encoder_to_native(e, io._heads_of(enc))
        else:
            native = io.text_encoder_to_native(e, io._heads_of(enc))
        for k, v in native.items():
            out["encoder." + k] = v
        for k, v in io.decoder_to_native(d, io._heads_of(dec), inter).items():
            out["decoder." + k] = v
        for a, b in (("generator.0.linear.weight", "generator.weight"), ("generator.0.linear.bias", "generator.bias")):
            if a in ref_sd:
                out[b] = ref_sd[a]
        if "generator.weight" not in out and "decoder.embed.weight" in out:
            out["generator.weight"] = out["decoder.embed.weight"]
        keys = set(target_keys) if target_keys is not None else None
        for k, v in ref_sd.items():       # native-named extras (CTC head, adapters ...)
            if k not in out and (keys is None or k in keys):
                out[k] = v
        return out


class SpeechToTextModel(Seq2SeqBase, _ReferenceNaming):
    """Audio encoder + text decoder with optional CTC head on the encoder states (``-ctc_loss``)."""

    def __init__(self, opt, encoder: nn.Module, decoder: nn.Module, vocab: int, generator_bias: bool = True, tie: bool = True):
        super().__init__()
        self.opt = opt
        self.encoder, self.decoder = encoder, decoder
        dim = decoder.embed.weight.shape[1]
        self.generator = Generator(dim, vocab, bias=generator_bias)
        if tie:
            self.tie_weights()
        self.pad_idx = decoder.embed.pad_idx
        self.label_smoothing = getattr(opt, "label_smoothing", 0.0)
        self.ctc_weight = getattr(opt, "ctc_loss", 0.0)
        # -ctc_loss_delay n: the CTC term joins the loss only once more than n updates have been made (the training
        # engine writes the optimiser's update count here; reference: onmt/train_utils/mp_trainer.py:795)
        self.ctc_delay = int(getattr(opt, "ctc_loss_delay", -1) if getattr(opt, "ctc_loss_delay", None) is not None else -1)
        self.num_updates = 0
        if self.ctc_weight > 0:
            self.ctc_linear = nn.Linear(encoder.dim, vocab)
        # -transducer_loss w: an RNN-T branch next to the attention decoder.  The decoder states act as the prediction
        # network, the joint is relu(f_t + g_u) -> Linear, blank = padding id (reference:
        # onmt/models/speech_recognizer/wav2vec2.py:557-566 construction, :697-730 loss)
        self.transducer_weight = float(getattr(opt, "transducer_loss", 0.0) or 0.0)
        if self.transducer_weight > 0:
            from ..ops.sequence import TransducerJoint, TransducerLoss
            if encoder.dim != dim:
                raise ValueError("-transducer_loss adds encoder and decoder states: their sizes must be equal")
            self.transducer_joint = TransducerJoint(pack_output=False, relu=True)
            self.transducer_linear = nn.Linear(dim, vocab)
            self.transducer_criterion = TransducerLoss(fuse_softmax_backward=False)

    # -predict_language: language-id heads on the encoder frames and on the decoder states, trained with a small weight
    # next to the translation loss (reference: onmt/train_utils/mp_trainer.py:834-846, 0.01 * (encoder + decoder term);
    # onmt/models/speech_recognizer/lid_loss.py:13)
    lid_weight = 0.01

    def enable_language_prediction(self, n_languages: int):
        self.n_languages = int(n_languages)
        self.enc_lid = nn.Linear(self.encoder.dim, self.n_languages)
        self.dec_lid = nn.Linear(self.decoder.embed.weight.shape[1], self.n_languages)

    @staticmethod
    def _per_row_language(lang, seqs, rows: int):
        """Per-sentence (or single) language ids -> one id per packed row."""
        from ..modules.dropout import _sentence_of_row
        lang = lang.view(-1).to(seqs.cu.device)
        sent = _sentence_of_row(seqs.cu, rows)
        return lang[sent] if lang.numel() > 1 else lang.expand(rows)

    def _lid_term(self, batch, context, src, out):
        tgt = out["tgt"]
        terms = []
        for head, states, seqs, key in ((self.enc_lid, context, src, "source_lang"), (self.dec_lid, out["hidden_packed"], tgt, "target_lang")):
            lang = batch.get(key) if hasattr(batch, "get") else None
            if lang is None:
                continue
            n = int(seqs.cu[-1])
            logits = head(states[:n].float())
            labels = self._per_row_language(lang, seqs, states.shape[0])[:n]
            terms.append(F.cross_entropy(logits, labels.long(), reduction="sum"))
        if not terms:
            return None
        out["lid_loss"] = sum(t.detach() for t in terms)
        return self.lid_weight * sum(terms)

    @torch.no_grad()
    def predict_language(self, batch):
        """Per-sentence language logits ``[B, n_languages]``: the encoder head's frame logits averaged over each utterance."""
        context, src = self.encode(batch)
        logp = torch.log_softmax(self.enc_lid(context.float()), -1)
        return src.pad(logp, time_first=False).sum(1) / (src.cu[1:] - src.cu[:-1]).clamp(min=1).unsqueeze(-1).float()

    def _transducer_term(self, context, src, out):
        tgt = out["tgt"]
        f = src.pad(context, time_first=False).float()                            # [B, T, H]
        g = tgt.pad(out["hidden_packed"], time_first=False).float()               # [B, U + 1, H]: states after BOS, y1 .. yU
        f_len = (src.cu[1:] - src.cu[:-1]).int()
        g_len = (tgt.cu[1:] - tgt.cu[:-1]).int()
        B = f.shape[0]
        tokens = tgt.pad(tgt.tokens[:, None].float(), time_first=False).squeeze(-1).long()    # [B, U + 1], BOS first
        labels = tokens[:, 1:].contiguous()                                        # y1 .. yU
        joint = self.transducer_joint(f, g, f_len[:B], g_len)
        logp = torch.log_softmax(self.transducer_linear(joint).float(), -1)       # [B, T, U + 1, V]
        loss = self.transducer_criterion(logp, labels, f_len[:B], g_len - 1, self.pad_idx)
        out["transducer_loss"], out["transducer_numel"] = loss.sum().detach(), int((g_len - 1).sum())
        return loss.sum()

    def encode(self, batch):
        if getattr(self.encoder, "adapters", None) is not None or getattr(self.encoder, "linear_proj", None) is not None:
            context, src = self.encoder(batch.get("source"), lang=single_language(batch, "source_lang"))
        else:
            context, src = self.encoder(batch.get("source"))
        self._uncompressed = None
        mode = str(getattr(self.opt, "ctc_compress", "None") or "None").lower()
        if mode != "none" and self.ctc_weight > 0:
            # merge runs of frames with the same CTC prediction before the decoder attends to them
            self._uncompressed = (context, src)
            logits = self.ctc_linear(context.float())
            context, src = ctc_compress(context, src, logits, mode)
        return context, src

    def auxiliary_losses(self, batch, context, src, out):
        if not self.training:
            return None
        extra = None
        if getattr(self, "enc_lid", None) is not None:
            extra = self._lid_term(batch, context, src, out)
        if self.transducer_weight > 0:
            if getattr(self, "_uncompressed", None) is not None:
                raise RuntimeError("-transducer_loss and -ctc_compress cannot be combined (the lattice needs every frame)")
            rnnt = self.transducer_weight * self._transducer_term(context, src, out)
            extra = rnnt if extra is None else extra + rnnt
        if self.ctc_weight <= 0 or self.num_updates <= self.ctc_delay:
            return extra
        ctc = self._ctc_term(batch, context, src, out)
        return ctc if extra is None else ctc + extra

    def _ctc_term(self, batch, context, src, out):
        if getattr(self, "_uncompressed", None) is not None:
            context, src = self._uncompressed              # the CTC loss is defined on the frame-level states
        logits = src.pad(self.ctc_linear(context.float()))                   # [T, B, V]
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        aux = batch.get("aux_target_output") if getattr(self, "ctc_on_aux", False) else None
        if aux is not None:
            # transcript side of a "triangle" corpus; its end-of-sentence symbol is not a CTC label
            targets = aux.t().clone()                                         # [B, U]
            last = batch.get("aux_tgt_lengths").to(targets.device) - 1
            targets[torch.arange(targets.shape[0], device=targets.device), last] = self.pad_idx
        else:
            targets = batch.get("target_output").t()                          # [B, U]
        tgt_len = (targets != self.pad_idx).sum(-1)
        lp = F.log_softmax(logits.float(), -1)
        ctc = F.ctc_loss(lp, targets, lengths[:targets.shape[0]], tgt_len, blank=self.pad_idx, reduction="sum", zero_infinity=True)
        out["ctc_loss"], out["n_ctc_targets"] = ctc.detach(), int(tgt_len.sum())
        return self.ctc_weight * ctc


class SpeechCTCModel(nn.Module):
    """``-no_decoder``: a speech encoder with a CTC output layer and nothing else (the reference builds its wav2vec 2.0
    models without a decoder under this flag, onmt/model_factory.py:274-276, and trains them on the CTC term alone).
    Blank is the padding id; the target's end-of-sentence symbol is not a label.  Decoding is the best path: arg-max
    per frame, repeats merged, blanks removed (``ctc_greedy``; the translator calls it instead of beam search)."""

    graph_capturable = False
    supports_logits_step = False
    ctc_only = True
    decoder = None

    def __init__(self, opt, encoder: nn.Module, vocab: int, pad_idx: int = 0, eos_idx: int = 3):
        super().__init__()
        self.opt, self.encoder = opt, encoder
        self.ctc_linear = nn.Linear(encoder.dim, vocab)
        self.pad_idx, self.eos_idx = pad_idx, eos_idx
        self.num_updates = 0

    def encode(self, batch):
        if getattr(self.encoder, "adapters", None) is not None or getattr(self.encoder, "linear_proj", None) is not None:
            return self.encoder(batch.get("source"), lang=single_language(batch, "source_lang"))
        return self.encoder(batch.get("source"))

    def _frame_logits(self, batch):
        context, src = self.encode(batch)
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        return src.pad(self.ctc_linear(context.float())), lengths                 # [T, B, V], [B]

    def forward(self, batch, grad_scale=None, **_unused) -> Dict:
        logits, lengths = self._frame_logits(batch)
        targets = batch.get("target_output").t().clone()                          # [B, U] ending in EOS
        targets[targets == self.eos_idx] = self.pad_idx
        tgt_len = (targets != self.pad_idx).sum(-1)
        lp = F.log_softmax(logits.float(), -1)
        ctc = F.ctc_loss(lp, targets, lengths[:targets.shape[0]], tgt_len, blank=self.pad_idx, reduction="sum", zero_infinity=True)
        loss = ctc if grad_scale is None else ctc * grad_scale
        return {"loss": loss, "ctc_loss": ctc.detach(), "n_ctc_targets": int(tgt_len.sum()),
                "correct": torch.zeros((), device=ctc.device), "row_loss": None}

    @torch.no_grad()
    def ctc_greedy(self, batch):
        """Best-path decoding: per utterance ``(token ids, sum of the chosen frames' log-probabilities)``."""
        logits, lengths = self._frame_logits(batch)
        lp = F.log_softmax(logits.float(), -1)
        best_lp, best = lp.max(-1)                                                # [T, B]
        out = []
        for b in range(best.shape[1]):
            n = int(lengths[b])
            path = best[:n, b]
            keep = torch.ones(n, dtype=torch.bool, device=path.device)
            keep[1:] = path[1:] != path[:-1]
            toks = path[keep & (path != self.pad_idx)]
            out.append((toks.tolist(), float(best_lp[:n, b].sum())))
        return out

    def create_decoder_state(self, *a, **kw):
        raise NotImplementedError("a model built with -no_decoder has no decoder to search with; use ctc_greedy (translate.py does)")


class TextToTextPretrained(Seq2SeqBase, _ReferenceNaming):
    """``pretrain_transformer``: pretrained-style text encoder + decoder (mBART, DeltaLM, M2M-100, BART ...)."""

    @property
    def graph_capturable(self):
        # reads only the packed token views - unless language adapters pick their weights by the batch's language id
        return getattr(self.decoder, "adapters", None) is None

    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        src_vocab, tgt_vocab = dicts["src"].size(), dicts["tgt"].size()
        efam, dfam = _encoder_family(opt), _decoder_family(opt)
        ecfg = load_json_config(getattr(opt, "enc_config_file", ""))
        dim = _cfg(ecfg, ["d_model", "encoder_embed_dim", "hidden_size"], opt.model_size)
        n_enc = opt.encoder_layers if getattr(opt, "encoder_layers", -1) > 0 else opt.layers
        self.encoder = PretrainedStyleEncoder(
            efam, _cfg(ecfg, ["vocab_size"], src_vocab), dim, _cfg(ecfg, ["encoder_layers", "num_hidden_layers"], n_enc),
            _cfg(ecfg, ["encoder_attention_heads", "num_attention_heads"], opt.n_heads),
            _cfg(ecfg, ["encoder_ffn_dim", "encoder_ffn_embed_dim", "intermediate_size"], opt.inner_size), opt.dropout,
            opt.attn_dropout, pad_idx=getattr(opt, "pad_idx", 1), layerdrop=getattr(opt, "death_rate", 0.0))
        self.decoder = build_pretrained_decoder(opt, tgt_vocab, dfam, kv_dim=dim)
        self.generator = Generator(self.decoder.embed.weight.shape[1], self.decoder.embed.weight.shape[0], bias=False)
        self.tie_weights()
        if getattr(opt, "join_embedding", False) and self.encoder.embed.weight.shape == self.decoder.embed.weight.shape:
            self.encoder.embed.weight = self.decoder.embed.weight
        self.pad_idx = self.decoder.embed.pad_idx
        self.label_smoothing = getattr(opt, "label_smoothing", 0.0)
        if int(getattr(opt, "decoder_adapter", 0) or 0) > 0:
            _add_language_adapters(opt, dicts, None, self.decoder)

    def encode(self, batch):
        src = batch.packed_source()
        return self.encoder(src), src


def _add_language_adapters(opt, dicts, encoder, decoder):
    from .transformer import _n_languages
    n = max(_n_languages(dicts), int(getattr(opt, "n_languages", 0) or 0))
    if encoder is not None and int(getattr(opt, "wav2vec_adapter", 0) or 0) > 0:
        if not hasattr(encoder, "add_adapters"):
            raise NotImplementedError("-wav2vec_adapter: %s has no adapter slots" % type(encoder).__name__)
        encoder.add_adapters(n, int(opt.wav2vec_adapter))
    if int(getattr(opt, "decoder_adapter", 0) or 0) > 0 and decoder is not None:
        if not hasattr(decoder, "add_adapters"):
            raise NotImplementedError("-decoder_adapter: %s has no adapter slots" % type(decoder).__name__)
        decoder.add_adapters(n, int(opt.decoder_adapter))


def _wav2vec_from_opt(opt):
    """Speech encoder chosen by substring of ``-enc_pretrained_model`` (reference: onmt/model_factory.py:247-272):
    ``s4`` -> state-space encoder on feature frames; ``w2vbert`` / ``w2v-bert`` / ``xeus`` -> Conformer-Shaw encoder on
    stacked filterbank frames (``models/w2vbert.py``); ``hubert`` / anything else -> the wav2vec 2.0 architecture on raw audio (HuBERT shares it);
    ``wavlm`` -> the same stack with the gated relative-position bias in every self-attention."""
    cfg = load_json_config(getattr(opt, "enc_config_file", ""))
    name = (getattr(opt, "enc_pretrained_model", "") or "wav2vec2").lower()
    if "s4" in name:
        from .mssm import build_stacked_mh_s4
        if getattr(opt, "s4_config_file", ""):          # -s4_config_file: the state-space sizes have a file of their own
            cfg = load_json_config(opt.s4_config_file)
        return build_stacked_mh_s4(getattr(opt, "input_size", 80), _cfg(cfg, ["encoder_embed_dim"], opt.model_size),
                                   _cfg(cfg, ["encoder_layers"], opt.layers), _cfg(cfg, ["num_heads"], 4),
                                   _cfg(cfg, ["state_dim"], 32), opt.dropout)
    if "w2vbert" in name or "w2v-bert" in name or "xeus" in name:
        from .w2vbert import build_w2vbert_encoder
        return build_w2vbert_encoder(opt, vars(cfg))
    base = "base" in name
    enc = Wav2Vec2Encoder(
        dim=_cfg(cfg, ["encoder_embed_dim", "hidden_size"], 768 if base else 1024),
        layers=_cfg(cfg, ["encoder_layers", "num_hidden_layers"], 12 if base else 24),
        heads=_cfg(cfg, ["encoder_attention_heads", "num_attention_heads"], 12 if base else 16),
        ffn=_cfg(cfg, ["encoder_ffn_embed_dim", "intermediate_size"], 3072 if base else 4096),
        dropout=getattr(opt, "enc_pretrain_hidden_dropout", opt.dropout) if hasattr(opt, "enc_pretrain_hidden_dropout") else opt.dropout,
        dropout_input=float(getattr(opt, "enc_pretrain_emb_dropout", 0.0) or 0.0),
        attn_dropout=opt.attn_dropout, layer_norm_first=_cfg(cfg, ["layer_norm_first"], not base),
        extractor_mode=_cfg(cfg, ["extractor_mode"], "default" if base else "layer_norm"),
        conv_bias=_cfg(cfg, ["conv_bias"], not base),
        mask_prob=getattr(opt, "wav2vec_spec_augment_mask_prob", 0.0) if hasattr(opt, "wav2vec_spec_augment_mask_prob") else 0.0,
        layerdrop=getattr(opt, "death_rate", 0.0) / 2,
        freeze_extractor=not getattr(opt, "unfreeze_feature_extractor", False),
        mask_channel_prob=0.2 if getattr(opt, "wav2vec_spec_augment", False) else 0.0,
        gated_relative_position="wavlm" in name,
        num_buckets=_cfg(cfg, ["num_buckets"], 320), max_distance=_cfg(cfg, ["max_distance"], 800))
    if getattr(opt, "wav2vec2_relative_attention", False) or getattr(opt, "add_relative_attention", False):
        # Transformer-XL style attention (sinusoidal relative positions, content and position biases) in every encoder
        # layer; its projections start from scratch next to the pretrained feed-forward blocks
        # (reference: onmt/models/speech_recognizer/wav2vec2.py:246-249 -> add_relative_attention)
        if "wavlm" in name or getattr(opt, "rotary_position_encoding", False):
            raise NotImplementedError("-wav2vec2_relative_attention excludes WavLM's bias and rotary positions")
        from .relative_transformer import RelativeSelfAttention
        for layer in enc.layers:
            layer.attn = RelativeSelfAttention(enc.dim, layer.attn.heads, opt.attn_dropout, causal=False)
    if getattr(opt, "rotary_position_encoding", False):
        # queries and keys of every encoder layer are rotated by their frame positions
        # (reference: onmt/models/speech_recognizer/wav2vec2.py:251-254 -> add_rotary_attention)
        if "wavlm" in name:
            raise NotImplementedError("-rotary_position_encoding and WavLM's relative-position bias exclude each other")
        for layer in enc.layers:
            layer.attn.rotary = True
    return enc


def _whisper_sizes(opt):
    cfg = load_json_config(getattr(opt, "dec_config_file", "") or getattr(opt, "enc_config_file", ""))
    return dict(dim=_cfg(cfg, ["d_model"], opt.model_size), enc_layers=_cfg(cfg, ["encoder_layers"], opt.layers),
                dec_layers=_cfg(cfg, ["decoder_layers"], opt.layers), heads=_cfg(cfg, ["encoder_attention_heads"], opt.n_heads),
                ffn=_cfg(cfg, ["encoder_ffn_dim"], opt.inner_size), n_mels=_cfg(cfg, ["num_mel_bins"], getattr(opt, "num_mel_bin", 80) or 80),
                src_pos=_cfg(cfg, ["max_source_positions"], 1500), tgt_pos=_cfg(cfg, ["max_target_positions"], 448),
                vocab=_cfg(cfg, ["vocab_size"], None), pad=_cfg(cfg, ["pad_token_id"], getattr(opt, "pad_idx", 0)))


def register_builders(register):
    @register("wav2vec2_bert", "quantize_wav2vec2_bert", "quantize_wav2vec2_mbart50")
    def _wav2vec_bert(opt, dicts):
        enc = _wav2vec_from_opt(opt)
        if getattr(opt, "no_decoder", False):
            _add_language_adapters(opt, dicts, enc, None)
            return SpeechCTCModel(opt, enc, dicts["tgt"].size(), getattr(opt, "pad_idx", 0))
        dec = build_pretrained_decoder(opt, dicts["tgt"].size(), kv_dim=enc.dim)
        _add_language_adapters(opt, dicts, enc, dec)
        return SpeechToTextModel(opt, enc, dec, dec.embed.weight.shape[0], generator_bias=False)

    @register("wav2vec2_transformer")
    def _wav2vec_transformer(opt, dicts):
        from .transformer import TransformerDecoder
        enc = _wav2vec_from_opt(opt)
        if getattr(opt, "no_decoder", False):
            return SpeechCTCModel(opt, enc, dicts["tgt"].size(), getattr(opt, "pad_idx", 0))
        embed = Embedding(dicts["tgt"].size(), opt.model_size, getattr(opt, "pad_idx", 0))
        dec = TransformerDecoder(opt, embed)
        if enc.dim != opt.model_size:
            for layer in dec.layers:
                layer.cross_attn.kv = type(layer.cross_attn.kv)(enc.dim, 2 * opt.model_size, bias=layer.cross_attn.kv.bias is not None)
        return SpeechToTextModel(opt, enc, dec, dicts["tgt"].size())

    @register("whisper")
    def _whisper(opt, dicts):
        s = _whisper_sizes(opt)
        vocab = s["vocab"] or dicts["tgt"].size()
        enc = WhisperEncoder(s["n_mels"], s["dim"], s["enc_layers"], s["heads"], s["ffn"], s["src_pos"], opt.dropout, opt.attn_dropout)
        dec = PretrainedStyleDecoder("whisper", vocab, s["dim"], s["dec_layers"], s["heads"], s["ffn"], opt.dropout,
                                     opt.attn_dropout, max_positions=s["tgt_pos"], pad_idx=s["pad"])
        return SpeechToTextModel(opt, enc, dec, vocab, generator_bias=False)

    @register("speech_transformer", "hybrid_transformer")
    def _speech_transformer(opt, dicts):
        from .transformer import TransformerDecoder, _n_languages
        opt.n_languages = max(_n_languages(dicts), int(getattr(opt, "n_languages", 0) or 0))
        enc = SpeechTransformerEncoder(opt, getattr(opt, "input_size", 40))
        embed = Embedding(dicts["tgt"].size(), opt.model_size, getattr(opt, "pad_idx", 0))
        dec = TransformerDecoder(opt, embed)
        return SpeechToTextModel(opt, enc, dec, dicts["tgt"].size())

    @register("pretrain_transformer", "deltalm", "mbart", "mbart50", "m2m100")
    def _pretrain_transformer(opt, dicts):
        return TextToTextPretrained(opt, dicts)
