"""Encoder-decoder Transformer (the ``-model transformer`` family) on packed variable-length batches.

Pre-LN layers, tensor2tensor sinusoidal positions added to ``sqrt(d) *`` word embeddings, optional joined
source/target embeddings and tied output projection, stochastic depth (``death_rate`` growing linearly
with depth), incremental decoding with per-layer key/value caches.  The forward pass never materialises
padded ``[T, B, H]`` activations or ``[T, B, V]`` logits in training: the trainer asks for the fused
``loss`` directly.  ``hidden`` / ``logprobs`` in the reference's padded layout are produced on request for
API parity.

Reference behaviour: onmt/models/transformers.py:48-223 (encoder), :226-510 (decoder, ``step`` :393),
:513-830 (``Transformer.forward`` :548, ``decode`` :685, ``step`` :754, ``create_decoder_state`` :792),
:833-999 (decoding state, ``_reorder_incremental_state`` :967); generator onmt/modules/base_seq2seq.py:8-47.
"""
from __future__ import annotations

import copy
import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from .. import ops
from ..modules.dropout import checkpointed
from .layers import DecoderLayer, Embedding, EncoderLayer, LayerNorm, PackedSeqs


def layer_structure_kwargs(opt) -> dict:
    """``-post_norm`` / ``-rezero`` / ``-macaron`` / ``-ffn_glu`` as keyword arguments of the shared layer classes."""
    return dict(post_norm=bool(getattr(opt, "post_norm", False)), rezero=bool(getattr(opt, "rezero", False)),
                macaron=bool(getattr(opt, "macaron", False)), glu=bool(getattr(opt, "ffn_glu", False)))


class LanguageEmbedding(nn.Module):
    """``-use_language_embedding``: one vector per language id, added to every position of a sentence
    (``-language_embedding_type sum | all_sum``) or concatenated and projected back (``concat``); reference:
    onmt/models/transformers.py:196-202 (encoder), :310-327 (decoder)."""

    def __init__(self, n_languages: int, dim: int, kind: str = "sum"):
        super().__init__()
        self.table = nn.Embedding(max(int(n_languages), 1), dim)
        nn.init.normal_(self.table.weight, 0.0, dim ** -0.5)
        self.kind = kind
        self.proj = nn.Linear(2 * dim, dim) if kind == "concat" else None

    def forward(self, x, seqs: PackedSeqs, lang_ids):
        """x ``[tokens, H]``; ``lang_ids`` ``[B]`` (or one id for the whole batch)."""
        if lang_ids is None:
            return x
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).to(torch.int64)
        ids = lang_ids.to(x.device).view(-1)
        if ids.numel() == 1:
            ids = ids.expand(lengths.numel())
        ids = ids[:lengths.numel()]
        if ids.numel() < lengths.numel():          # static batch capacity: the extra sentences are empty
            ids = torch.cat([ids, ids.new_zeros(lengths.numel() - ids.numel())])
        per_token = torch.repeat_interleave(self.table(ids), lengths, dim=0, output_size=None)
        if per_token.shape[0] < x.shape[0]:        # rows past the last sentence of a packed buffer
            per_token = torch.cat([per_token, per_token.new_zeros(x.shape[0] - per_token.shape[0], per_token.shape[1])])
        if self.kind == "concat":
            return self.proj(torch.cat([x.float(), per_token.float()], dim=-1)).to(x.dtype)
        return x + per_token.to(x.dtype)


def _n_languages(dicts) -> int:
    langs = dicts.get("langs") if hasattr(dicts, "get") else None
    return len(langs) if langs else 1


def single_language(batch, key: str) -> Optional[int]:
    """The one language id of a batch (batches of the multilingual data sets hold one language pair each), or None."""
    t = batch.get(key) if hasattr(batch, "get") else None
    if t is None or not torch.is_tensor(t) or t.numel() == 0:
        return None
    return int(t.view(-1)[0])


def _embed_with_language(stack, seqs: PackedSeqs, lang_ids):
    """Embedding (+ language vector) + embedding dropout.  Without language embeddings this is the one fused kernel."""
    if stack.language_embedding is None or lang_ids is None:
        return stack.embed(seqs, stack.emb_dropout)
    x = stack.language_embedding(stack.embed(seqs, 0.0), seqs, lang_ids)
    return ops.dropout_add(x.contiguous(), None, stack.emb_dropout, stack.training)


def _apply_regularisation_options(stack, opt, side: str = "enc"):
    """``-variational_dropout`` (time-shared masks on the residual branches), ``-word_dropout`` (vocabulary-level
    dropout in the embedding), ``-checkpointing N`` (recompute the first N layers in backward) and
    ``-enc_gradient_checkpointing`` / ``-dec_gradient_checkpointing`` (recompute every layer of that stack)."""
    stack.checkpointing = int(getattr(opt, "checkpointing", 0) or 0)
    whole_stack = getattr(opt, "enc_gradient_checkpointing", False) if side == "enc" else getattr(opt, "dec_gradient_checkpointing", False)
    if whole_stack:
        stack.checkpointing = 10 ** 6
    for layer in stack.layers:
        layer.variational = bool(getattr(opt, "variational_dropout", False))
    stack.embed.word_dropout = float(getattr(opt, "word_dropout", 0.0) or 0.0)


def _expected_death_rates(n_layers: int, death_rate: float):
    return [(i + 1) / n_layers * death_rate for i in range(n_layers)]


class TransformerEncoder(nn.Module):
    def __init__(self, opt, embed: Embedding):
        super().__init__()
        n = opt.encoder_layers if getattr(opt, "encoder_layers", -1) > 0 else opt.layers
        self.embed = embed
        self.emb_dropout = opt.emb_dropout
        rates = _expected_death_rates(n, getattr(opt, "death_rate", 0.0))
        self.layers = nn.ModuleList([
            EncoderLayer(opt.model_size, opt.n_heads, opt.inner_size, opt.dropout, opt.attn_dropout, opt.ffn_activation,
                         attn_bias=getattr(opt, "attn_bias", False), death_rate=rates[i],
                         ffn_dropout=opt.ffn_dropout if getattr(opt, "ffn_dropout", -1) >= 0 else None,
                         **layer_structure_kwargs(opt))
            for i in range(n)])
        self.final_norm = LayerNorm(opt.model_size)
        self.language_embedding = None
        _apply_regularisation_options(self, opt, "enc")
        self.reversible = None
        if getattr(opt, "src_reversible", False):
            # activations are reconstructed in backward instead of stored (reference: onmt/reversible_models)
            from .reversible import ReversibleStack
            self.layers = nn.ModuleList()
            self.reversible = ReversibleStack(n, opt.model_size, opt.n_heads, opt.inner_size, opt.dropout, opt.attn_dropout,
                                              opt.ffn_activation)

    def forward(self, src: PackedSeqs, lang_ids=None):
        x = _embed_with_language(self, src, lang_ids)
        if self.reversible is not None:
            return self.reversible(x, src)
        for i, layer in enumerate(self.layers):
            if self.training and i < self.checkpointing:
                x = checkpointed(layer, x, src)
            else:
                x = layer(x, src)
        return self.final_norm(x)


class TransformerDecoder(nn.Module):
    def __init__(self, opt, embed: Embedding, ignore_source: bool = False):
        super().__init__()
        self.embed = embed
        self.emb_dropout = opt.emb_dropout
        # -death_rate_decoder overrides the shared -death_rate for this stack
        dr = getattr(opt, "death_rate_decoder", 0.0) or getattr(opt, "death_rate", 0.0)
        rates = _expected_death_rates(opt.layers, dr)
        self.layers = nn.ModuleList([
            DecoderLayer(opt.model_size, opt.n_heads, opt.inner_size, opt.dropout, opt.attn_dropout, opt.ffn_activation,
                         attn_bias=getattr(opt, "attn_bias", False), death_rate=rates[i],
                         ffn_dropout=opt.ffn_dropout if getattr(opt, "ffn_dropout", -1) >= 0 else None,
                         ignore_source=ignore_source, **layer_structure_kwargs(opt))
            for i in range(opt.layers)])
        self.final_norm = LayerNorm(opt.model_size)
        self.language_embedding = None
        _apply_regularisation_options(self, opt, "dec")
        self.reversible = None
        if getattr(opt, "tgt_reversible", False) and not ignore_source:
            from .reversible import ReversibleStack
            self.n_layers = opt.layers
            self.layers = nn.ModuleList()
            self.reversible = ReversibleStack(opt.layers, opt.model_size, opt.n_heads, opt.inner_size, opt.dropout,
                                              opt.attn_dropout, opt.ffn_activation, causal=True, cross=True)
            self.layers = self.reversible.layers      # decoding state set-up walks the layers (cross-attention caches)

    def forward(self, tgt: PackedSeqs, memory, src: PackedSeqs, lang_ids=None):
        x = _embed_with_language(self, tgt, lang_ids)
        if self.reversible is not None:
            return self.reversible(x, tgt, memory, src)
        for i, layer in enumerate(self.layers):
            if self.training and i < self.checkpointing:
                x = checkpointed(layer, x, tgt, memory, src)
            else:
                x = layer(x, tgt, memory, src)
        return self.final_norm(x)

    def step(self, tokens, position: int, state: "DecodingState"):
        """tokens [B] (last generated symbol of every hypothesis) -> hidden [B, H]."""
        B = tokens.shape[0]
        seqs = PackedSeqs(tokens, torch.full_like(tokens, position), torch.arange(B + 1, dtype=torch.int32, device=tokens.device), 1)
        self.embed.renew(position + 1)
        x = self.embed(seqs, 0.0)
        if self.language_embedding is not None and getattr(state, "tgt_lang", None) is not None:
            x = self.language_embedding(x, seqs, state.tgt_lang)
        return self.run_layers_step(x, state)

    def run_layers_step(self, x, state: "DecodingState"):
        """One new position through the layer stack (subclasses with a different wiring override this)."""
        if self.reversible is not None:
            return self.reversible.step(x, state.buffers, state.src_pad_mask)
        for i, layer in enumerate(self.layers):
            x = layer.step(x, state.buffers[i], state.src_pad_mask)
        return self.final_norm(x)

    def step_static(self, tokens, positions, state: "DecodingState"):
        """``step`` with the positions given as a device tensor and no host-side bookkeeping, so that the whole call
        can be captured in a CUDA graph (``state.enable_device_positions()`` must have been called)."""
        B = tokens.shape[0]
        cu = getattr(self, "_step_cu", None)
        if cu is None or cu.numel() != B + 1 or cu.device != tokens.device:
            cu = self._step_cu = torch.arange(B + 1, dtype=torch.int32, device=tokens.device)
        return self.run_layers_step(self.embed(PackedSeqs(tokens, positions, cu, 1), 0.0), state)


class Generator(nn.Module):
    """hidden -> vocabulary logits (weight optionally tied to the target embedding)."""

    def __init__(self, dim: int, vocab: int, bias: bool = True, fix_norm: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim))
        nn.init.normal_(self.weight, 0.0, dim ** -0.5)
        self.bias = nn.Parameter(torch.zeros(vocab)) if bias else None
        self.fix_norm = fix_norm      # -fix_norm_output_embedding: unit-length output embeddings (base_seq2seq.py:33-41)

    def forward(self, hidden, log_softmax: bool = False):
        if self.fix_norm:
            w = torch.nn.functional.normalize(self.weight.float(), dim=-1).to(hidden.dtype)
            logits = torch.nn.functional.linear(hidden, w, None if self.bias is None else self.bias.to(hidden.dtype))
            return torch.log_softmax(logits.float(), dim=-1) if log_softmax else logits
        logits = ops.linear(hidden, self.weight, self.bias, "none", 0.0, None, False)
        return torch.log_softmax(logits.float(), dim=-1) if log_softmax else logits


class DecodingState:
    """Encoder output (padded once, repeated per beam) plus per-layer key/value caches.

    ``buffers[i]`` holds ``k``/``v`` (self-attention, grown by one position per step) and ``c_k``/``c_v``
    (projected encoder states, computed once).  ``reorder`` re-indexes every tensor along the hypothesis
    dimension, which is what beam search needs after each step.
    """

    def __init__(self, context_padded, src_pad_mask, n_layers: int, beam_size: int):
        self.beam_size = beam_size
        self.context = context_padded.repeat_interleave(beam_size, 0) if beam_size > 1 else context_padded
        self.src_pad_mask = src_pad_mask.repeat_interleave(beam_size, 0) if beam_size > 1 else src_pad_mask
        self.buffers = [dict() for _ in range(n_layers)]
        self.position = 0

    def set_cache_capacity(self, cap: int):
        """Ask the self-attention layers for preallocated ``[rows, cap, H]`` key/value caches (CUDA bf16 path)."""
        for buf in self.buffers:
            buf["cap"] = int(cap)

    def enable_device_positions(self):
        """Keep the write position of the self-attention caches in a device integer (``pos_dev``) that the caller
        advances once per step, so that a decoding step can be captured in a CUDA graph and replayed."""
        self.pos_dev = torch.zeros(1, dtype=torch.int32, device=self.context.device)
        for buf in self.buffers:
            buf["pos_dev"] = self.pos_dev

    def reorder(self, index, reorder_context: bool = True):
        rows = index.numel()
        if reorder_context:
            self.context = self.context.index_select(0, index)
            self.src_pad_mask = self.src_pad_mask.index_select(0, index)
            if getattr(self, "src_tokens", None) is not None:
                self.src_tokens = self.src_tokens.index_select(0, index)
        for buf in self.buffers:
            if "k_spare" in buf and buf.get("pos_dev") is not None:
                H = buf["k"].shape[2]
                ops.ext().gather_rows(buf["k"], buf["k_spare"], index, -1, buf["pos_dev"], H)
                ops.ext().gather_rows(buf["v"], buf["v_spare"], index, -1, buf["pos_dev"], H)
                buf["k"], buf["k_spare"] = buf["k_spare"], buf["k"]
                buf["v"], buf["v_spare"] = buf["v_spare"], buf["v"]
            elif "k_spare" in buf:
                # preallocated caches: copy only the filled prefix of every row into the spare buffers and swap
                filled = buf.get("pos", 0) * buf["k"].shape[2]
                ops.ext().gather_rows(buf["k"], buf["k_spare"], index, filled)
                ops.ext().gather_rows(buf["v"], buf["v_spare"], index, filled)
                buf["k"], buf["k_spare"] = buf["k_spare"], buf["k"]
                buf["v"], buf["v_spare"] = buf["v_spare"], buf["v"]
            for k in list(buf.keys()):
                val = buf[k]
                if k == "pos_dev" or (k in ("k", "v", "k_spare", "v_spare") and "k_spare" in buf):
                    continue
                # per-sentence entries (encoder-decoder caches shared by the hypotheses) keep their order
                if torch.is_tensor(val) and val.dim() > 0 and val.shape[0] == rows:
                    buf[k] = val.index_select(0, index)

    _reorder_incremental_state = reorder  # reference spelling


class Seq2SeqBase(nn.Module):
    """Shared behaviour of every encoder-decoder model: fused training loss, gold scoring, incremental decoding.

    Subclasses provide ``encode(batch) -> (context_packed [Ns, H], src PackedSeqs)``, ``self.decoder`` (forward on
    packed targets + ``step``) and ``self.generator``; everything trainers and translators call lives here
    (model contract of the reference: onmt/models/transformers.py:548-830, onmt/modules/base_seq2seq.py:50-150).
    """

    pad_idx = 0
    label_smoothing = 0.0
    generator_chunk_rows = 0      # > 0: output projection + loss over this many rows at a time (no [rows, V] logits)

    # A captured training step reads nothing but the packed token views of a batch from fixed device buffers.  A model
    # whose forward pass depends on anything else of the batch (language ids, audio features, auxiliary targets) or on
    # state carried between steps must leave this False; the engine then runs it kernel by kernel.
    graph_capturable = False

    def encode(self, batch):
        raise NotImplementedError

    def auxiliary_losses(self, batch, context, src, out):
        """Hook for CTC / language-id / contrastive terms; returns a tensor to add to the loss or None."""
        return None

    switchout = 0.0

    def _switchout(self, seqs: PackedSeqs, vocab: int) -> PackedSeqs:
        from ..modules.dropout import switchout_packed
        return PackedSeqs(switchout_packed(seqs.tokens, seqs.cu, vocab, self.switchout), seqs.positions, seqs.cu, seqs.max_len,
                          seqs.lengths, seqs.extras)

    def forward(self, batch, return_logits: bool = False, compute_loss: bool = True, grad_scale=None, **_unused) -> Dict:
        context, src = self.encode(batch)
        tgt = batch.packed_target_input()
        if self.training and self.switchout > 0:
            tgt = self._switchout(tgt, self.generator.weight.shape[0])
        labels = batch.packed_target_output()
        if getattr(self.decoder, "language_embedding", None) is not None:
            hidden = self.decoder(tgt, context, src, lang_ids=batch.get("target_lang") if hasattr(batch, "get") else None)
        elif getattr(self.decoder, "adapters", None) is not None:
            hidden = self.decoder(tgt, context, src, lang=single_language(batch, "target_lang"))
        else:
            hidden = self.decoder(tgt, context, src)
        out = {"hidden_packed": hidden, "context_packed": context, "src": src, "tgt": tgt, "target": labels}
        if compute_loss and self.training and getattr(self, "nce", None) is not None:
            # noise-contrastive training: target and noise scores only, no [rows, V] logits
            res = self.nce_loss(self.nce(hidden, labels), labels)
            loss = res["loss"]
            if grad_scale is not None and torch.is_grad_enabled():
                from ..ops.reference import scale_gradient
                gs = grad_scale if isinstance(grad_scale, torch.Tensor) else torch.tensor(float(grad_scale), device=loss.device)
                loss = scale_gradient(loss, gs.to(loss.device))
            out.update(loss=loss, correct=None, row_loss=None)
        elif compute_loss and getattr(self, "copy_generator", None) is not None:
            # padded, unfused: the copy distribution needs the [B, T, S] attention of every target position over its source
            logp = self._copy_log_probs(tgt.pad(hidden, time_first=False), context, src)          # [B, T, V]
            gold = tgt.pad(labels[:, None].float(), time_first=False).squeeze(-1).long()            # [B, T]
            valid = gold != self.pad_idx
            nll = -logp.gather(-1, gold.clamp(min=0)[..., None]).squeeze(-1)
            eps = self.label_smoothing if self.training else 0.0
            tok = (1.0 - eps) * nll - eps * logp.mean(-1) if eps > 0 else nll
            loss = (tok * valid).sum().reshape(1)
            if grad_scale is not None and torch.is_grad_enabled():
                from ..ops.reference import scale_gradient
                gs = grad_scale if isinstance(grad_scale, torch.Tensor) else torch.tensor(float(grad_scale), device=loss.device)
                loss = scale_gradient(loss, gs.to(loss.device))
            correct = ((logp.argmax(-1) == gold) & valid).sum().float().reshape(1)
            out.update(loss=loss, correct=correct, row_loss=None)
        elif compute_loss and getattr(self.generator, "fix_norm", False):
            logits = self.generator(hidden)
            loss, correct, row_loss = ops.cross_entropy(logits if logits.is_contiguous() else logits.contiguous(), labels,
                                                        self.label_smoothing if self.training else 0.0, self.pad_idx)
            if grad_scale is not None and torch.is_grad_enabled():
                from ..ops.reference import scale_gradient
                gs = grad_scale if isinstance(grad_scale, torch.Tensor) else torch.tensor(float(grad_scale), device=loss.device)
                loss = scale_gradient(loss, gs.to(loss.device))
            out.update(loss=loss, correct=correct, row_loss=row_loss)
        elif compute_loss:
            loss, correct, row_loss = ops.generator_cross_entropy(
                hidden, self.generator.weight, self.generator.bias, labels,
                self.label_smoothing if self.training else 0.0, self.pad_idx, grad_scale,
                chunk_rows=self.generator_chunk_rows if self.training else 0)
            out.update(loss=loss, correct=correct, row_loss=row_loss)
        if compute_loss:
            aux = self.auxiliary_losses(batch, context, src, out)
            if aux is not None:
                out["nmt_loss"] = out["loss"]
                out["loss"] = out["loss"] + aux
        if return_logits:
            logits = self.generator(hidden)
            out["logprobs"] = tgt.pad(logits)       # [T, B, V] (logits, as in the reference)
            out["hidden"] = tgt.pad(hidden)         # [T, B, H]
            out["context"] = src.pad(context)
            lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
            out["src_mask"] = torch.arange(src.max_len, device=lengths.device)[None, :] >= lengths[:, None]   # [B, Ts], True = padding
            out["target_mask"] = batch.get("target_input_selfattn_mask") if hasattr(batch, "get") else None
            out["softmaxed"] = False
        return out

    def _copy_log_probs(self, hidden_bt, context, src):
        ctx = src.pad(context, time_first=False)                                   # [B, S, H]
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        pad = torch.arange(ctx.shape[1], device=ctx.device)[None, :] >= lengths[:, None]
        toks = src.pad(src.tokens[:, None].float(), time_first=False).squeeze(-1).long()
        B = hidden_bt.shape[0]
        return self.copy_generator(hidden_bt, ctx[:B], toks[:B], pad[:B])

    def load_encoder_weights(self, pretrained, strict: bool = False):
        """Copy the encoder of another model (a module, or a checkpoint's ``model`` state dict) into this one; used to
        start a speech-translation or continual-learning run from a trained encoder
        (reference: onmt/models/transformers.py ``load_encoder_weights``)."""
        state = pretrained.state_dict() if isinstance(pretrained, nn.Module) else pretrained
        if any(k.startswith("encoder.") for k in state):
            state = {k[len("encoder."):]: v for k, v in state.items() if k.startswith("encoder.")}
        return self.encoder.load_state_dict(state, strict=strict)

    def init_stream(self):
        """Streaming state for models with segment memories; models without one decode sentence by sentence."""
        return None

    def post_backward(self, output_dict=None):
        return None

    def tie_weights(self):
        self.generator.weight = self.decoder.embed.weight

    @torch.no_grad()
    def decode(self, batch):
        """Gold scoring: per-sentence sum of target log-probabilities ``[B]`` and per-token scores ``[T, B]``."""
        was_training = self.training
        self.eval()
        out = self.forward(batch, compute_loss=True)
        padded = out["tgt"].pad((-out["row_loss"])[:, None]).squeeze(-1)
        self.train(was_training)
        return batch.get("target_output"), padded.sum(0), padded

    @torch.no_grad()
    def create_decoder_state(self, batch, beam_size: int = 1, **_unused) -> DecodingState:
        context, src = self.encode(batch)
        ctx_padded = src.pad(context, time_first=False)                    # [B, Ts, H]
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        pad_mask = torch.arange(ctx_padded.shape[1], device=ctx_padded.device)[None, :] >= lengths[:, None]
        state = DecodingState(ctx_padded, pad_mask, len(self.decoder.layers), beam_size)
        if getattr(self, "copy_generator", None) is not None:
            toks = src.pad(src.tokens[:, None].float(), time_first=False).squeeze(-1).long()[:ctx_padded.shape[0]]
            state.src_tokens = toks.repeat_interleave(beam_size, 0) if beam_size > 1 else toks
        if (getattr(self.decoder, "language_embedding", None) is not None
                or getattr(self.decoder, "adapters", None) is not None) and hasattr(batch, "get"):
            tl = batch.get("target_lang")
            if tl is not None:
                tl = tl.to(ctx_padded.device).view(-1)
                state.tgt_lang = tl.repeat_interleave(beam_size, 0) if (beam_size > 1 and tl.numel() > 1) else tl
        shared = ctx_padded.is_cuda and ctx_padded.dtype == torch.bfloat16 and beam_size > 1
        for i, layer in enumerate(self.decoder.layers):
            if not getattr(layer, "ignore_source", False):
                # on the GPU the projected encoder states are kept once per sentence, not once per hypothesis
                ck, cv = layer.cross_attn.precompute(ctx_padded if shared else state.context)
                state.buffers[i]["c_k"], state.buffers[i]["c_v"] = ck, cv
                if ctx_padded.is_cuda and ctx_padded.dtype == torch.bfloat16:
                    state.buffers[i]["c_len"] = lengths.to(torch.int32).contiguous()
        return state

    supports_logits_step = True

    @torch.no_grad()
    def step(self, input_t, state: DecodingState, logits_only: bool = False) -> Dict:
        """input_t ``[B*beam, t]`` (all symbols so far) -> ``log_prob [B*beam, V]`` fp32 for the next symbol
        (``logits_only``: raw ``logits`` instead, for the fused log-softmax + top-k beam kernel)."""
        tokens = input_t[:, -1].contiguous()
        hidden = self.decoder.step(tokens, input_t.shape[1] - 1, state)
        if getattr(self, "copy_generator", None) is not None and getattr(state, "src_tokens", None) is not None:
            state.position += 1
            logp = self.copy_generator(hidden[:, None, :], state.context, state.src_tokens, state.src_pad_mask).squeeze(1)
            return {"log_prob": logp, "logits": logp, "hidden": hidden, "coverage": None}
        logits = self.generator(hidden)
        state.position += 1
        if logits_only:
            return {"logits": logits, "hidden": hidden, "coverage": None}
        return {"log_prob": torch.log_softmax(logits.float(), dim=-1), "hidden": hidden, "coverage": None}

    def renew_buffer(self, new_len: int):
        for m in (getattr(self, "encoder", None), getattr(self, "decoder", None)):
            emb = getattr(m, "embed", None)
            if emb is not None and hasattr(emb, "renew"):
                emb.renew(new_len)


class Transformer(Seq2SeqBase):
    """``NMTModel`` for text-to-text translation."""

    @property
    def graph_capturable(self):
        # language embeddings read the batch's language ids, which the static buffers of a captured step do not carry
        return getattr(self.decoder, "language_embedding", None) is None

    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        src_vocab, tgt_vocab = dicts["src"].size(), dicts["tgt"].size()
        self.pad_idx = getattr(opt, "pad_idx", 0)
        max_pos = getattr(opt, "max_position_length", 1024)
        tgt_embed = Embedding(tgt_vocab, opt.model_size, self.pad_idx, max_pos=max_pos)
        if getattr(opt, "join_embedding", False):
            assert src_vocab == tgt_vocab, "joined embeddings need one shared vocabulary"
            src_embed = Embedding(src_vocab, opt.model_size, self.pad_idx, max_pos=max_pos)
            src_embed.weight = tgt_embed.weight
        else:
            src_embed = Embedding(src_vocab, opt.model_size, self.pad_idx, max_pos=max_pos)
        self.encoder = TransformerEncoder(opt, src_embed)
        self.decoder = TransformerDecoder(opt, tgt_embed)
        self.generator = Generator(opt.model_size, tgt_vocab, fix_norm=bool(getattr(opt, "fix_norm_output_embedding", False)))
        if getattr(opt, "use_language_embedding", False):
            lang = LanguageEmbedding(_n_languages(dicts), opt.model_size, getattr(opt, "language_embedding_type", "sum"))
            self.encoder.language_embedding = lang
            self.decoder.language_embedding = lang       # one table for both sides, as in the reference's factory
        if getattr(opt, "tie_weights", False):
            self.tie_weights()
        self.label_smoothing = getattr(opt, "label_smoothing", 0.0)
        self.switchout = float(getattr(opt, "switchout", 0.0) or 0.0)
        self.generator_chunk_rows = int(getattr(opt, "generator_chunk_rows", 0) or 0)
        # -mirror_loss: a second decoder reads the target right to left; its loss is added and the forward decoder's
        # states (through a learned map g) are pulled towards the backward decoder's states of the same positions
        if float(getattr(opt, "transducer_loss", 0.0) or 0.0) > 0:
            raise NotImplementedError("-transducer_loss is built for the speech models (frames against labels); "
                                      "the text Transformer has no transducer branch")
        self.mirror_weight = float(getattr(opt, "mirror_loss", 0.0) or 0.0)
        if self.mirror_weight > 0:
            self.mirror_decoder = copy.deepcopy(self.decoder)
            self.mirror_g = nn.Linear(opt.model_size, opt.model_size)
            self.mirror_generator = Generator(opt.model_size, tgt_vocab)
            self.mirror_generator.weight = self.decoder.embed.weight
        # nce_noise > 0 (set by older checkpoints' options): noise-contrastive training of the output layer
        if int(getattr(opt, "nce_noise", 0) or 0) > 0:
            from ..modules.nce import NCELinear, NCELoss, build_unigram_noise
            self.nce = NCELinear(opt.model_size, tgt_vocab, build_unigram_noise(dictionary=dicts["tgt"]), int(opt.nce_noise),
                                 weight=self.generator.weight, bias=self.generator.bias if self.generator.bias is not None else False)
            self.nce_loss = NCELoss(opt.model_size, tgt_vocab, int(opt.nce_noise), label_smoothing=self.label_smoothing,
                                    padding_idx=self.pad_idx)
        # -copy_generator: output distribution mixed with a copy distribution over the source words (one shared vocabulary)
        if getattr(opt, "copy_generator", False):
            if src_vocab != tgt_vocab:
                raise ValueError("-copy_generator needs one shared vocabulary (-join_vocab): copied source words are target words")
            from ..modules.copy_generator import CopyGenerator
            self.copy_generator = CopyGenerator(opt.model_size, tgt_vocab, weight=self.generator.weight,
                                                fix_norm=bool(getattr(opt, "fix_norm_output_embedding", False)))
            self.supports_logits_step = False      # decoding goes through the mixed distribution, not raw logits
        # -reconstruct: a third decoder regenerates the source from the decoder's states
        self.reconstruct = bool(getattr(opt, "reconstruct", False))
        if self.reconstruct:
            rec_embed = Embedding(src_vocab, opt.model_size, self.pad_idx, max_pos=max_pos)
            rec_embed.weight = self.encoder.embed.weight
            self.rec_linear = nn.Linear(opt.model_size, opt.model_size)
            self.rec_decoder = TransformerDecoder(opt, rec_embed)
            self.rec_generator = Generator(opt.model_size, src_vocab)
            self.rec_generator.weight = self.encoder.embed.weight

    @staticmethod
    def _flip_index(seqs: PackedSeqs, rows: int):
        """Row permutation that reverses every sequence of a packed batch in place (rows of the static padding map to
        themselves)."""
        from ..modules.dropout import _sentence_of_row
        cu = seqs.cu.to(torch.int64)
        sent = _sentence_of_row(seqs.cu, rows)
        i = torch.arange(rows, device=cu.device)
        flipped = cu[sent] + cu[sent + 1] - 1 - i
        return torch.where(i < cu[-1], flipped, i)

    def auxiliary_losses(self, batch, context, src, out):
        """Mirror network and source reconstruction (reference: onmt/models/transformers.py:622-666 for the extra
        decoders, onmt/modules/loss.py:321-391 for the terms).  With the full target ``BOS y1 .. yn EOS`` the backward
        decoder's input is the per-sentence reversal of the forward labels and its labels are the reversal of the forward
        inputs; the state of the backward decoder at reversed position t is the regression target (no gradient) of
        ``g(forward state t)``, summed squared error divided by the model size."""
        if not self.training or not (self.mirror_weight > 0 or self.reconstruct):
            return None
        tgt, hidden, labels = out["tgt"], out["hidden_packed"], out["target"]
        smoothing = self.label_smoothing
        total = None
        if self.mirror_weight > 0:
            rows = tgt.tokens.shape[0]
            flip = self._flip_index(tgt, rows)
            rev_in = PackedSeqs(labels.index_select(0, flip), tgt.positions, tgt.cu, tgt.max_len, tgt.lengths, tgt.extras)
            rev_labels = tgt.tokens.index_select(0, flip)
            rev_labels = torch.where(labels == self.pad_idx, torch.full_like(rev_labels, self.pad_idx), rev_labels)
            rev_hidden = self.mirror_decoder(rev_in, context, src)
            rev_loss, _, _ = ops.generator_cross_entropy(rev_hidden, self.mirror_generator.weight, self.mirror_generator.bias,
                                                         rev_labels, smoothing, self.pad_idx)
            valid = (labels != self.pad_idx).unsqueeze(-1)
            target_states = rev_hidden.detach().index_select(0, flip)
            diff = (self.mirror_g(hidden).float() - target_states.float()) * valid
            mirror = diff.pow(2).sum() / hidden.shape[-1]
            out["rev_loss"], out["mirror_loss"] = rev_loss.detach(), mirror.detach()
            total = rev_loss + self.mirror_weight * mirror
        if self.reconstruct:
            # input of the reconstruction decoder: the source shifted right behind the target's first symbol (BOS)
            n = src.tokens.shape[0]
            cu = src.cu.to(torch.int64)
            shifted = torch.cat([src.tokens[:1], src.tokens[:-1]])
            first = torch.zeros(n, dtype=torch.bool, device=src.tokens.device)
            first[cu[:-1].clamp(max=n - 1)] = True
            bos = tgt.tokens[tgt.cu[:-1].to(torch.int64)][0]
            rec_in = PackedSeqs(torch.where(first, bos.expand(n), shifted), src.positions, src.cu, src.max_len, src.lengths, src.extras)
            rec_hidden = self.rec_decoder(rec_in, self.rec_linear(hidden), tgt)
            rec_loss, _, _ = ops.generator_cross_entropy(rec_hidden, self.rec_generator.weight, self.rec_generator.bias,
                                                         src.tokens, smoothing, self.pad_idx)
            out["rec_loss"] = rec_loss.detach()
            total = rec_loss if total is None else total + rec_loss
        return total

    def share_enc_dec_embedding(self):
        self.encoder.embed.weight = self.decoder.embed.weight

    def encode(self, batch):
        src = batch.packed_source()
        if self.training and self.switchout > 0:
            src = self._switchout(src, self.encoder.embed.weight.shape[0])
        if self.encoder.language_embedding is not None:
            return self.encoder(src, lang_ids=batch.get("source_lang") if hasattr(batch, "get") else None), src
        return self.encoder(src), src
