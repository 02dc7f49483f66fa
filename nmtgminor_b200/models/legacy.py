"""The older model zoo, rebuilt on the packed layers so that its checkpoints' model names keep working.

* ``DlclTransformer`` — dynamic linear combination of layers: the input of layer l+1 is a learned mix of the
  layer-normalised outputs of the embedding and of all layers up to l
  (reference: onmt/legacy/DynamicTransformer/Dlcl.py:15-174, Models.py:10-140).
* ``ParallelTransformer`` — decoder layer i attends to the normalised output of encoder layer i instead of the
  top of the encoder (onmt/legacy/ParallelTransformer/Models.py:95-158, 310-372).
* ``FCTransformer`` — "fully connected": every decoder layer attends uniformly over the states of ALL encoder layers;
  the memory bank of a sentence is its L layer outputs laid end to end
  (onmt/legacy/FCTransformer/Layers.py:23-145 ``UniformMultiHeadAttention``, Models.py:19-308).
* ``UnifiedTransformer`` — one causal stack over ``[source ; target]`` with language-model masking; the loss is taken on
  the target part (onmt/legacy/old_models/unified_transformer.py:17-200).
* ``FusionNetwork`` — a translation model with a frozen language model added to its logits ("cold fusion", pre-norm
  variant: ``log_softmax(tm_logits + log p_lm)``; onmt/legacy/FusionNetwork/Models.py:10-196).
* ``LSTMLanguageModel`` — stacked LSTM language model (onmt/legacy/LSTMLM/Models.py:21-297).

``distance_transformer`` and ``memory_transformer`` of the reference are relative-position models with a learnable
distance table / segment memory; those names are served by ``models/relative_transformer.py``.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import DecoderLayer, Embedding, LayerNorm, PackedSeqs
from .transformer import (DecodingState, Generator, Seq2SeqBase, Transformer, TransformerDecoder, TransformerEncoder,
                          _expected_death_rates)


# ------------------------------------------------------------------------------------------------------------
class DynamicLinearCombination(nn.Module):
    """x_{l+1} = sum_{k<=l} W[l, k] * LN_k(y_k) with a learnable lower-triangular W (rows initialised to the average;
    ``normalize`` divides each row by its sum so the mix stays an average while it is learned)."""

    def __init__(self, dim: int, n_layers: int, init: str = "avg", normalize: bool = True):
        super().__init__()
        n = n_layers + 1
        w = torch.zeros(n, n)
        for i in range(n):
            if init == "one":
                w[i, i] = 1.0
            else:
                w[i, :i + 1] = 1.0 / (i + 1)
        self.weight = nn.Parameter(w)
        self.register_buffer("mask", torch.tril(torch.ones(n, n)), persistent=False)
        self.norms = nn.ModuleList([nn.Identity()] + [LayerNorm(dim) for _ in range(n - 1)])
        self.normalize = normalize

    def push(self, history: List[torch.Tensor], y: torch.Tensor) -> None:
        history.append(self.norms[len(history)](y))

    def pop(self, history: List[torch.Tensor]) -> torch.Tensor:
        i = len(history) - 1
        w = (self.weight[i] * self.mask[i])[:i + 1]
        if self.normalize:
            w = w / w.sum()
        out = history[0] * w[0].to(history[0].dtype)
        for k in range(1, i + 1):
            out = out + history[k] * w[k].to(history[k].dtype)
        return out


class DlclEncoder(TransformerEncoder):
    def __init__(self, opt, embed):
        super().__init__(opt, embed)
        self.history = DynamicLinearCombination(opt.model_size, len(self.layers))

    def forward(self, src: PackedSeqs):
        hist: List[torch.Tensor] = []
        self.history.push(hist, self.embed(src, self.emb_dropout))
        for layer in self.layers:
            self.history.push(hist, layer(self.history.pop(hist), src))
        return self.history.pop(hist)       # already normalised per state: no extra final norm


class DlclDecoder(TransformerDecoder):
    def __init__(self, opt, embed):
        super().__init__(opt, embed)
        self.history = DynamicLinearCombination(opt.model_size, len(self.layers))

    def forward(self, tgt: PackedSeqs, memory, src: PackedSeqs):
        hist: List[torch.Tensor] = []
        self.history.push(hist, self.embed(tgt, self.emb_dropout))
        for layer in self.layers:
            self.history.push(hist, layer(self.history.pop(hist), tgt, memory, src))
        return self.history.pop(hist)

    def run_layers_step(self, x, state):
        hist: List[torch.Tensor] = []
        self.history.push(hist, x)
        for i, layer in enumerate(self.layers):
            self.history.push(hist, layer.step(self.history.pop(hist), state.buffers[i], state.src_pad_mask))
        return self.history.pop(hist)


class DlclTransformer(Transformer):
    def __init__(self, opt, dicts):
        super().__init__(opt, dicts)
        self.encoder = DlclEncoder(opt, self.encoder.embed)
        self.decoder = DlclDecoder(opt, self.decoder.embed)


# ------------------------------------------------------------------------------------------------------------
class _BankEncoder(TransformerEncoder):
    """Encoder that also returns the per-layer memory bank: the normalised input of layers 2..L plus the final output."""

    def __init__(self, opt, embed):
        super().__init__(opt, embed)
        self.bank_norms = nn.ModuleList([LayerNorm(opt.model_size) for _ in range(max(len(self.layers) - 1, 0))])

    def forward_bank(self, src: PackedSeqs):
        x = self.embed(src, self.emb_dropout)
        bank = []
        for i, layer in enumerate(self.layers):
            x = layer(x, src)
            if i + 1 < len(self.layers):
                bank.append(self.bank_norms[i](x))
        bank.append(self.final_norm(x))
        return bank


class ParallelDecoder(TransformerDecoder):
    def forward(self, tgt: PackedSeqs, memory, src: PackedSeqs):
        bank = src.extras["memory_bank"]
        x = self.embed(tgt, self.emb_dropout)
        for i, layer in enumerate(self.layers):
            x = layer(x, tgt, bank[min(i, len(bank) - 1)], src)
        return self.final_norm(x)


class ParallelTransformer(Transformer):
    def __init__(self, opt, dicts):
        super().__init__(opt, dicts)
        self.encoder = _BankEncoder(opt, self.encoder.embed)
        self.decoder = ParallelDecoder(opt, self.decoder.embed)

    def encode(self, batch):
        src = batch.packed_source()
        bank = self.encoder.forward_bank(src)
        src = PackedSeqs(src.tokens, src.positions, src.cu, src.max_len, src.lengths, dict(src.extras, memory_bank=bank))
        return bank[-1], src

    @torch.no_grad()
    def create_decoder_state(self, batch, beam_size: int = 1, **_unused) -> DecodingState:
        context, src = self.encode(batch)
        bank = src.extras["memory_bank"]
        top = src.pad(context, time_first=False)
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        pad_mask = torch.arange(top.shape[1], device=top.device)[None, :] >= lengths[:, None]
        state = DecodingState(top, pad_mask, len(self.decoder.layers), beam_size)
        shared = top.is_cuda and top.dtype == torch.bfloat16 and beam_size > 1
        for i, layer in enumerate(self.decoder.layers):
            ctx = src.pad(bank[min(i, len(bank) - 1)], time_first=False)
            if not shared and beam_size > 1:
                ctx = ctx.repeat_interleave(beam_size, 0)
            state.buffers[i]["c_k"], state.buffers[i]["c_v"] = layer.cross_attn.precompute(ctx)
            if top.is_cuda and top.dtype == torch.bfloat16:
                state.buffers[i]["c_len"] = lengths.to(torch.int32).contiguous()
        return state


# ------------------------------------------------------------------------------------------------------------
def layer_major_bank(bank: List[torch.Tensor], src: PackedSeqs):
    """L packed ``[Ns, H]`` layer outputs -> one packed memory in which sentence b owns ``L * len_b`` consecutive rows
    (layer 0's states, then layer 1's, ...), with the matching ``PackedSeqs`` descriptor."""
    L = len(bank)
    cap = bank[0].shape[0]
    cu = src.cu.to(torch.int64)
    lengths = cu[1:] - cu[:-1]
    rows = torch.arange(cap, device=bank[0].device)
    seq = torch.searchsorted(cu[1:].contiguous(), rows, right=True).clamp(max=lengths.numel() - 1)
    valid = rows < cu[-1]
    offset = rows - cu[seq]
    out = bank[0].new_zeros((L * cap, bank[0].shape[1]))
    for l, states in enumerate(bank):
        dest = L * cu[seq] + l * lengths[seq] + offset
        dest = torch.where(valid, dest, torch.full_like(dest, L * cap - 1))   # rows past the batch land on a spare row
        out = out.index_copy(0, dest, states * valid[:, None].to(states.dtype))
    new_cu = (cu * L).to(torch.int32)
    positions = torch.zeros(L * cap, dtype=torch.long, device=out.device)
    tokens = torch.zeros(L * cap, dtype=torch.long, device=out.device)
    return out, PackedSeqs(tokens, positions, new_cu, src.max_len * L, lengths * L)


class FCTransformer(Transformer):
    def __init__(self, opt, dicts):
        super().__init__(opt, dicts)
        self.encoder = _BankEncoder(opt, self.encoder.embed)

    def encode(self, batch):
        src = batch.packed_source()
        return layer_major_bank(self.encoder.forward_bank(src), src)


# ------------------------------------------------------------------------------------------------------------
def _join_source_target(src: PackedSeqs, tgt: PackedSeqs):
    """Concatenate sentence b of ``src`` and of ``tgt`` into one sequence; returns the joint descriptor and, for every
    target row, its row in the joint layout."""
    dev = src.tokens.device
    scu, tcu = src.cu.to(torch.int64), tgt.cu.to(torch.int64)
    slen, tlen = scu[1:] - scu[:-1], tcu[1:] - tcu[:-1]
    jcu = torch.zeros_like(scu)
    jcu[1:] = torch.cumsum(slen + tlen, 0)
    ns, nt = int(scu[-1]), int(tcu[-1])
    srow = torch.arange(ns, device=dev)
    sseq = torch.searchsorted(scu[1:].contiguous(), srow, right=True)
    s_dest = jcu[sseq] + (srow - scu[sseq])
    trow = torch.arange(nt, device=dev)
    tseq = torch.searchsorted(tcu[1:].contiguous(), trow, right=True)
    t_off = trow - tcu[tseq]
    t_dest = jcu[tseq] + slen[tseq] + t_off
    n = ns + nt
    tokens = torch.zeros(n, dtype=torch.long, device=dev)
    positions = torch.zeros(n, dtype=torch.long, device=dev)
    tokens[s_dest] = src.tokens[:ns]
    tokens[t_dest] = tgt.tokens[:nt]
    positions[s_dest] = src.positions[:ns]
    positions[t_dest] = t_off
    joint = PackedSeqs(tokens, positions, jcu.to(torch.int32), src.max_len + tgt.max_len, slen + tlen)
    is_src = torch.zeros(n, dtype=torch.bool, device=dev)
    is_src[s_dest] = True
    return joint, t_dest, is_src


class _UnifiedState:
    """Decoding state of the joint stack: the source tokens (the model re-reads ``[source ; prefix]`` every step)."""

    def __init__(self, src_tokens, src_lengths, beam_size):
        self.src_tokens = src_tokens.repeat_interleave(beam_size, 0)
        self.src_lengths = src_lengths.repeat_interleave(beam_size, 0)
        self.position = 0

    @property
    def context(self):
        return self.src_tokens

    @property
    def src_pad_mask(self):
        return torch.arange(self.src_tokens.shape[1], device=self.src_tokens.device)[None, :] >= self.src_lengths[:, None]

    def reorder(self, index, reorder_context: bool = True):
        self.src_tokens = self.src_tokens.index_select(0, index)
        self.src_lengths = self.src_lengths.index_select(0, index)


class UnifiedTransformer(Seq2SeqBase):
    supports_logits_step = False

    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        src_vocab, tgt_vocab = dicts["src"].size(), dicts["tgt"].size()
        self.pad_idx = getattr(opt, "pad_idx", 0)
        max_pos = getattr(opt, "max_position_length", 1024)
        self.tgt_embed = Embedding(tgt_vocab, opt.model_size, self.pad_idx, max_pos=max_pos)
        self.src_embed = Embedding(src_vocab, opt.model_size, self.pad_idx, max_pos=max_pos)
        if getattr(opt, "join_embedding", False) or src_vocab == tgt_vocab:
            self.src_embed.weight = self.tgt_embed.weight
        rates = _expected_death_rates(opt.layers, getattr(opt, "death_rate", 0.0))
        self.layers = nn.ModuleList([
            DecoderLayer(opt.model_size, opt.n_heads, opt.inner_size, opt.dropout, opt.attn_dropout, opt.ffn_activation,
                         death_rate=rates[i], ignore_source=True) for i in range(opt.layers)])
        self.final_norm = LayerNorm(opt.model_size)
        self.generator = Generator(opt.model_size, tgt_vocab)
        if getattr(opt, "tie_weights", False):
            self.generator.weight = self.tgt_embed.weight
        self.emb_dropout = opt.emb_dropout
        self.label_smoothing = getattr(opt, "label_smoothing", 0.0)

    def renew_buffer(self, new_len: int):
        self.src_embed.renew(new_len)
        self.tgt_embed.renew(new_len)

    def _hidden(self, src: PackedSeqs, tgt: PackedSeqs):
        joint, t_dest, is_src = _join_source_target(src, tgt)
        p = self.emb_dropout if self.training else 0.0
        e_src = self.src_embed(joint, p)
        if self.src_embed.weight is self.tgt_embed.weight:
            x = e_src
        else:
            x = torch.where(is_src[:, None], e_src, self.tgt_embed(joint, p))
        for layer in self.layers:
            x = layer(x, joint, None, None)
        return self.final_norm(x).index_select(0, t_dest)

    def forward(self, batch, return_logits: bool = False, compute_loss: bool = True, grad_scale=None, **_unused) -> Dict:
        src, tgt = batch.packed_source(), batch.packed_target_input()
        nt = int(tgt.cu[-1])
        hidden = self._hidden(src, tgt)
        labels = batch.packed_target_output()[:nt]
        out = {"hidden_packed": hidden, "src": src, "tgt": tgt, "target": labels}
        if compute_loss:
            loss, correct, row_loss = ops.generator_cross_entropy(
                hidden, self.generator.weight, self.generator.bias, labels,
                self.label_smoothing if self.training else 0.0, self.pad_idx, grad_scale)
            if row_loss.shape[0] < tgt.tokens.shape[0]:
                row_loss = F.pad(row_loss, (0, tgt.tokens.shape[0] - row_loss.shape[0]))
            out.update(loss=loss, correct=correct, row_loss=row_loss)
        if return_logits:
            logits = self.generator(hidden)
            full = logits.new_zeros((tgt.tokens.shape[0], logits.shape[1]))
            full[:nt] = logits
            out["logprobs"] = tgt.pad(full)
        return out

    @torch.no_grad()
    def create_decoder_state(self, batch, beam_size: int = 1, **_unused):
        src = batch.packed_source()
        lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        padded = src.pad(src.tokens[:, None], time_first=False).squeeze(-1)
        return _UnifiedState(padded, lengths, beam_size)

    @torch.no_grad()
    def step(self, input_t, state, logits_only: bool = False) -> Dict:
        R, t = input_t.shape
        src = PackedSeqs.from_padded(state.src_tokens, state.src_lengths, pad_idx=self.pad_idx)
        tgt = PackedSeqs.from_padded(input_t, torch.full((R,), t, dtype=torch.int64, device=input_t.device), pad_idx=self.pad_idx)
        hidden = self._hidden(src, tgt)
        last = hidden.view(R, t, -1)[:, -1]
        logits = self.generator(last)
        state.position += 1
        return {"log_prob": torch.log_softmax(logits.float(), dim=-1), "hidden": last, "coverage": None}


# ------------------------------------------------------------------------------------------------------------
class LSTMLanguageModel(nn.Module):
    """Embedding -> stacked LSTM -> (tied) output layer; trained on ``target_input`` -> ``target_output``."""

    def __init__(self, opt, dicts):
        super().__init__()
        vocab = dicts["tgt"].size()
        self.pad_idx = getattr(opt, "pad_idx", 0)
        self.embed = nn.Embedding(vocab, opt.model_size, padding_idx=self.pad_idx)
        self.rnn = nn.LSTM(opt.model_size, opt.model_size, num_layers=opt.layers, dropout=opt.dropout if opt.layers > 1 else 0.0)
        self.drop = nn.Dropout(opt.dropout)
        self.generator = Generator(opt.model_size, vocab)
        if getattr(opt, "tie_weights", False):
            self.generator.weight = self.embed.weight
        self.label_smoothing = getattr(opt, "label_smoothing", 0.0)

    def hidden_states(self, tokens_tb, state=None):
        out, state = self.rnn(self.drop(self.embed(tokens_tb)), state)
        return self.drop(out), state

    def forward(self, batch, grad_scale=None, **_unused) -> Dict:
        inp, gold = batch.get("target_input"), batch.get("target_output")
        hidden, _ = self.hidden_states(inp)
        logits = self.generator(hidden.reshape(-1, hidden.shape[-1])).float()
        loss, correct, row_loss = ops.cross_entropy(logits, gold.reshape(-1), self.label_smoothing if self.training else 0.0,
                                                    self.pad_idx)
        return {"loss": loss, "correct": correct, "row_loss": row_loss, "hidden": hidden, "target": gold}

    @torch.no_grad()
    def log_probs(self, tokens_tb):
        """Next-token log-probabilities ``[T, B, V]`` for a prefix matrix (used by ``FusionNetwork``)."""
        hidden, _ = self.hidden_states(tokens_tb)
        return torch.log_softmax(self.generator(hidden.reshape(-1, hidden.shape[-1])).float(), -1).view(*tokens_tb.shape, -1)


class FusionNetwork(nn.Module):
    """Translation model + frozen language model: ``log p = log_softmax(tm_logits + log p_lm)``.

    The language model may be any module with ``log_probs(tokens [T, B]) -> [T, B, V]`` over the target vocabulary
    (``LSTMLanguageModel`` here); its parameters never receive gradients."""

    supports_logits_step = False

    def __init__(self, tm_model, lm_model):
        super().__init__()
        self.tm_model, self.lm_model = tm_model, lm_model
        for p in self.lm_model.parameters():
            p.requires_grad_(False)
        self.pad_idx = getattr(tm_model, "pad_idx", 0)

    @property
    def decoder(self):
        return None      # no graph-captured decoder step: the search calls ``step``

    def forward(self, batch, **kw) -> Dict:
        out = self.tm_model(batch, compute_loss=False, return_logits=True, **{k: v for k, v in kw.items() if k == "grad_scale"})
        self.lm_model.eval()
        log_lm = self.lm_model.log_probs(batch.get("target_input"))                 # [T, B, V]
        fused = torch.log_softmax(out["logprobs"].float() + log_lm, dim=-1)
        gold = batch.get("target_output")
        smoothing = self.tm_model.label_smoothing if self.training else 0.0
        flat, g = fused.reshape(-1, fused.shape[-1]), gold.reshape(-1)
        keep = g != self.pad_idx
        nll = -flat.gather(1, g[:, None]).squeeze(1)
        if smoothing > 0:
            nll = (1 - smoothing) * nll - smoothing * flat.mean(-1)
        row_loss = nll * keep
        out.update(loss=row_loss.sum(), correct=((flat.argmax(-1) == g) & keep).sum(), row_loss=row_loss, tm=out.get("logprobs"),
                   lm=log_lm)
        return out

    def renew_buffer(self, n):
        self.tm_model.renew_buffer(n)

    @torch.no_grad()
    def create_decoder_state(self, batch, beam_size: int = 1, **kw):
        return self.tm_model.create_decoder_state(batch, beam_size, **kw)

    @torch.no_grad()
    def step(self, input_t, state, logits_only: bool = False) -> Dict:
        tm = self.tm_model.step(input_t, state, logits_only=True)
        log_lm = self.lm_model.log_probs(input_t.t().contiguous())[-1]
        return {"log_prob": torch.log_softmax(tm["logits"].float() + log_lm, dim=-1), "hidden": tm["hidden"], "coverage": None}

    @torch.no_grad()
    def decode(self, batch):
        was = self.training
        self.eval()
        out = self.forward(batch)
        T, B = batch.get("target_output").shape
        per_tok = (-out["row_loss"]).view(T, B)
        self.train(was)
        return batch.get("target_output"), per_tok.sum(0), per_tok


def register_builders(register):
    register("dlcl_transformer", "dynamic_transformer")(lambda opt, dicts: DlclTransformer(opt, dicts))
    register("parallel_transformer")(lambda opt, dicts: ParallelTransformer(opt, dicts))
    register("fctransformer", "fc_transformer")(lambda opt, dicts: FCTransformer(opt, dicts))
    register("unified_transformer")(lambda opt, dicts: UnifiedTransformer(opt, dicts))
    register("lstm_lm")(lambda opt, dicts: LSTMLanguageModel(opt, dicts))

    def _relative(opt, dicts):
        from .relative_transformer import RelativeTransformer
        opt.learnable_position_encoding = True          # the "distance" models learn their relative-position table
        return RelativeTransformer(opt, dicts)
    register("distance_transformer", "memory_transformer", "relative_unified_transformer")(_relative)
