"""Output layer that can copy source words: ``p(w) = (1 - z) softmax(W h)[w] + z * sum_{j: src_j = w} a_j`` with the copy
gate ``z = sigmoid(w_z . h)`` and the copy distribution ``a = softmax_j(h . c_j)`` over the encoder states ``c`` of the
sentence.  Source and target must share one vocabulary (``-join_vocab``): a source word is copied by adding its attention
mass to its own entry of the output distribution.

``forward(hidden [B, T, H], context [B, S, H], src_tokens [B, S], src_pad_mask [B, S]) -> log p [B, T, V]`` (fp32).

Reference: onmt/modules/copy_generator.py:10-134 (gate :91, scatter of the copy mass :118), model_factory.py:123-130.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class CopyGenerator(nn.Module):
    def __init__(self, hidden_size: int, output_size: int, weight: Optional[nn.Parameter] = None, fix_norm: bool = False):
        super().__init__()
        self.hidden_size, self.output_size, self.fix_norm = hidden_size, output_size, fix_norm
        self.linear_copy = nn.Linear(hidden_size, 1)
        nn.init.xavier_uniform_(self.linear_copy.weight)
        self.linear = nn.Linear(hidden_size, output_size)
        stdv = 1.0 / math.sqrt(hidden_size)
        nn.init.uniform_(self.linear.weight, -stdv, stdv)
        if weight is not None:
            self.linear.weight = weight                       # tied to the target embedding
        self.must_softmax = True

    def forward(self, hidden, context, src_tokens, src_pad_mask=None, log: bool = True):
        h = hidden.float()
        z = torch.sigmoid(self.linear_copy(h))                                       # [B, T, 1]
        w = F.normalize(self.linear.weight.float(), dim=-1) if self.fix_norm else self.linear.weight.float()
        p_gen = torch.softmax(F.linear(h, w, self.linear.bias.float()), dim=-1) * (1.0 - z)
        score = torch.bmm(h, context.float().transpose(1, 2))                        # [B, T, S]
        if src_pad_mask is not None:
            score = score.masked_fill(src_pad_mask[:, None, :], float("-inf"))
        attn = torch.softmax(score, dim=-1)
        p_copy = attn * z
        if src_pad_mask is not None:
            p_copy = p_copy.masked_fill(src_pad_mask[:, None, :], 0.0)
        idx = src_tokens.clamp(0, self.output_size - 1)[:, None, :].expand(-1, h.shape[1], -1)
        p = p_gen.scatter_add(2, idx, p_copy)
        return torch.log(p.clamp_min(1e-30)) if log else p
