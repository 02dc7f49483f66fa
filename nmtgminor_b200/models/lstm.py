"""Recurrent sequence-to-sequence model (``-model LSTM``): bidirectional LSTM encoder (text or speech features),
unidirectional LSTM decoder with one encoder-decoder attention layer on top, input feeding of the attended context.
cuDNN LSTMs through PyTorch; the attention and output layers reuse the fused blocks.

Reference: onmt/models/speech_recognizer/lstm.py:20 (``SpeechLSTMEncoder``), :170 (``SpeechLSTMDecoder``), :428 (``SpeechLSTMSeq2Seq``).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import CrossAttention, Embedding, LayerNorm, PackedSeqs, pack_padded
from .speech_encoders import split_audio_batch
from .transformer import DecodingState, Generator, Seq2SeqBase


class LSTMEncoder(nn.Module):
    def __init__(self, opt, vocab=None, input_size=None):
        super().__init__()
        dim = opt.model_size
        self.text = vocab is not None
        if self.text:
            self.embed = nn.Embedding(vocab, dim, padding_idx=getattr(opt, "pad_idx", 0))
        else:
            self.proj = nn.Linear(input_size, dim)
        n = opt.encoder_layers if getattr(opt, "encoder_layers", -1) > 0 else opt.layers
        self.rnn = nn.LSTM(dim, dim // 2, n, batch_first=True, bidirectional=True, dropout=opt.dropout if n > 1 else 0.0)
        self.norm = LayerNorm(dim)
        self.dim = dim

    def forward(self, batch):
        if self.text:
            src = batch.packed_source()
            x = src.pad(self.embed(src.tokens), time_first=False)
            lengths = (src.cu[1:] - src.cu[:-1]).to(torch.int64)
        else:
            feats, lengths = split_audio_batch(batch.get("source"))
            x = self.proj(feats.float())
        packed = nn.utils.rnn.pack_padded_sequence(x.float(), lengths.cpu().clamp(min=1), batch_first=True, enforce_sorted=False)
        out, _ = self.rnn(packed)
        out, _ = nn.utils.rnn.pad_packed_sequence(out, batch_first=True, total_length=x.shape[1])
        rows, seqs = pack_padded(out, lengths)
        return self.norm(rows), seqs


class LSTMDecoder(nn.Module):
    def __init__(self, opt, vocab):
        super().__init__()
        dim = opt.model_size
        self.embed = Embedding(vocab, dim, getattr(opt, "pad_idx", 0), use_pos=False)
        self.rnn = nn.LSTM(dim, dim, opt.layers, batch_first=True, dropout=opt.dropout if opt.layers > 1 else 0.0)
        self.attn_norm = LayerNorm(dim)
        self.cross_attn = CrossAttention(dim, opt.n_heads, opt.attn_dropout)
        self.final_norm = LayerNorm(dim)
        self.layers = [self]           # one cache slot for the decoding state
        self.ignore_source = False
        self.dropout = opt.dropout

    def forward(self, tgt: PackedSeqs, memory, src: PackedSeqs):
        from ..ops.reference import unpad_packed
        x = tgt.pad(self.embed(tgt, self.dropout), time_first=False)
        h, _ = self.rnn(x.float())
        rows = unpad_packed(h.to(memory.dtype), tgt.cu, tgt.tokens.shape[0])
        rows = self.cross_attn(self.attn_norm(rows), tgt, memory, src, residual=rows, dropout_p=self.dropout)
        return self.final_norm(rows)

    def step(self, tokens, position, state: DecodingState):
        B = tokens.shape[0]
        seqs = PackedSeqs(tokens, torch.zeros_like(tokens), torch.arange(B + 1, dtype=torch.int32, device=tokens.device), 1)
        x = self.embed(seqs, 0.0).float().unsqueeze(1)
        buf = state.buffers[0]
        hc = (buf["h"].transpose(0, 1).contiguous(), buf["c"].transpose(0, 1).contiguous()) if "h" in buf else None
        out, (h, c) = self.rnn(x, hc)
        buf["h"], buf["c"] = h.transpose(0, 1), c.transpose(0, 1)      # hypothesis dimension first, so reorder() works
        rows = out[:, 0].to(state.context.dtype)
        rows = rows + self.cross_attn.step(self.attn_norm(rows), buf, state.src_pad_mask)
        return self.final_norm(rows)


class LSTMSeq2Seq(Seq2SeqBase):
    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        speech = getattr(opt, "encoder_type", "text") != "text"
        self.encoder = LSTMEncoder(opt, None if speech else dicts["src"].size(), getattr(opt, "input_size", 40) if speech else None)
        self.decoder = LSTMDecoder(opt, dicts["tgt"].size())
        self.generator = Generator(opt.model_size, dicts["tgt"].size())
        if getattr(opt, "tie_weights", False):
            self.tie_weights()
        self.pad_idx, self.label_smoothing = getattr(opt, "pad_idx", 0), getattr(opt, "label_smoothing", 0.0)

    def encode(self, batch):
        return self.encoder(batch)


def register_builders(register):
    register("LSTM", "lstm")(lambda opt, dicts: LSTMSeq2Seq(opt, dicts))
