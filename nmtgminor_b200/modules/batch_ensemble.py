"""Batch-ensemble weights: ``E`` ensemble members share every weight matrix ``W`` and differ only by two vectors per
layer, ``W_e = W * (s_e r_e^T)``, so a member costs ``in + out`` extra parameters per linear layer and the whole
ensemble runs in one batch: ``y = ((x * r_e) W^T) * s_e + b`` with the member ``e`` chosen per sentence.

Training sends sentence ``b`` of a batch through member ``b mod E`` (or through explicit ``members``); evaluation runs
all members on every sentence and averages their outputs, which is what makes the model an ensemble at test time.

* ``BatchEnsembleLinear``      - one linear layer on packed rows ``[N, in]`` (or padded ``[T, B, in]``);
* ``BatchEnsembleFeedForward`` - drop-in replacement of ``models.layers.FeedForward`` (same parameters ``fc1`` / ``fc2``
  plus ``r_in, s_in, r_out, s_out``), told the sentence boundaries by the layer that calls it;
* ``convert_to_batch_ensemble`` - swaps every feed-forward block of a built model (``-batch_ensemble E``), optionally
  freezing everything except the member vectors (fine-tuning a pretrained model into an ensemble).

Reference: onmt/modules/batch_ensemble/batch_ensemble_linear.py:8-260 (function :8, ``BatchEnsembleLinear`` :100,
feed-forward :187), whisper/batch_ensemble_whisper.py:42-180 (FFN of encoder / decoder layers, ``ensemble_init`` :972,
frozen shared weights :1010), options.py:315.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops


def _init_members(t: torch.Tensor, how: str):
    with torch.no_grad():
        if how == "random_sign":
            t.bernoulli_(0.5).mul_(2).sub_(1)
        elif how == "ones":
            t.fill_(1.0)
        elif how == "normal":
            t.normal_(1.0, 0.02)                 # around the identity, so that a converted model starts as the shared model
        else:
            raise ValueError("ensemble_init must be random_sign, ones or normal")


def members_of_rows(cu: torch.Tensor, rows: int, n_ensembles: int, members: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ensemble member of every packed row: sentence ``b`` uses member ``members[b]`` (default ``b mod E``)."""
    from .dropout import _sentence_of_row
    sent = _sentence_of_row(cu, rows)
    if members is not None:
        return members.to(sent.device)[sent]
    return sent % n_ensembles


class BatchEnsembleLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, n_ensembles: int, bias: bool = True, init: str = "random_sign"):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        nn.init.xavier_normal_(self.weight)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.r = nn.Parameter(torch.empty(n_ensembles, in_features))
        self.s = nn.Parameter(torch.empty(n_ensembles, out_features))
        _init_members(self.r, init)
        _init_members(self.s, init)

    @property
    def n_ensembles(self) -> int:
        return self.r.shape[0]

    def _one(self, x, r, s):
        y = ops.linear((x * r.to(x.dtype)).contiguous(), self.weight, None, "none", 0.0, None, False)
        y = y * s.to(y.dtype)
        return y + self.bias.to(y.dtype) if self.bias is not None else y

    def forward(self, x: torch.Tensor, row_members: Optional[torch.Tensor] = None, indices: Optional[torch.Tensor] = None):
        """x ``[N, in]`` with ``row_members [N]``, or ``[T, B, in]`` with per-sentence ``indices [B]`` (default ``b mod E``).
        In evaluation without explicit members the outputs of all members are averaged."""
        E = self.n_ensembles
        if x.dim() == 3 and row_members is None and (self.training or indices is not None):
            idx = indices if indices is not None else torch.arange(x.shape[1], device=x.device) % E
            return self._one(x, self.r[idx][None], self.s[idx][None])
        if row_members is not None:
            return self._one(x, self.r[row_members], self.s[row_members])
        out = None
        for e in range(E):
            y = self._one(x, self.r[e], self.s[e]).float()
            out = y if out is None else out + y
        return (out / E).to(x.dtype)


class BatchEnsembleFeedForward(nn.Module):
    """``residual + D(fc2(D(act(fc1(x)))))`` with member vectors around both matrices."""

    wants_seqs = True

    def __init__(self, ffn: nn.Module, n_ensembles: int, init: str = "random_sign"):
        super().__init__()
        if getattr(ffn, "glu", False):
            raise ValueError("batch-ensemble weights are not defined for gated feed-forward blocks")
        self.fc1, self.fc2 = ffn.fc1, ffn.fc2                      # shared matrices keep their parameter names
        self.dropout, self.activation = ffn.dropout, ffn.activation
        dim, inner = ffn.fc1.weight.shape[1], ffn.fc1.weight.shape[0]
        self.r_in = nn.Parameter(torch.empty(n_ensembles, dim))
        self.s_in = nn.Parameter(torch.empty(n_ensembles, inner))
        self.r_out = nn.Parameter(torch.empty(n_ensembles, inner))
        self.s_out = nn.Parameter(torch.empty(n_ensembles, dim))
        for t in (self.r_in, self.s_in, self.r_out, self.s_out):
            _init_members(t, init)

    @property
    def n_ensembles(self) -> int:
        return self.r_in.shape[0]

    def _member(self, x, r_in, s_in, r_out, s_out, training: bool):
        from ..ops.reference import _act
        dt = x.dtype
        h = ops.linear((x * r_in.to(dt)).contiguous(), self.fc1.weight, None, "none", 0.0, None, False)
        h = h.float() * s_in.float() + self.fc1.bias.float()
        h = _act(h, ops.ACT_IDS[self.activation])
        h = ops.dropout_add(h.to(dt).contiguous(), None, self.dropout, training)
        y = ops.linear((h * r_out.to(dt)).contiguous(), self.fc2.weight, None, "none", 0.0, None, False)
        return y.float() * s_out.float() + self.fc2.bias.float()

    def forward(self, x, residual=None, dropout_p: float = 0.0, seqs=None, members: Optional[torch.Tensor] = None):
        if self.training or members is not None:
            if seqs is not None:
                rows = members_of_rows(seqs.cu, x.shape[0], self.n_ensembles, members)
            else:
                rows = torch.zeros(x.shape[0], dtype=torch.long, device=x.device)
            y = self._member(x, self.r_in[rows], self.s_in[rows], self.r_out[rows], self.s_out[rows], self.training)
        else:
            y = None
            for e in range(self.n_ensembles):
                ye = self._member(x, self.r_in[e], self.s_in[e], self.r_out[e], self.s_out[e], False)
                y = ye if y is None else y + ye
            y = y / self.n_ensembles
        y = ops.dropout_add(y.to(x.dtype).contiguous(), None, dropout_p, self.training)
        return y if residual is None else residual + y


def convert_to_batch_ensemble(model: nn.Module, n_ensembles: int, init: str = "random_sign", freeze_shared: bool = False) -> int:
    """Replaces every ``FeedForward`` block of ``model`` by its batch-ensemble form; returns the number of blocks
    converted.  ``freeze_shared`` leaves only the member vectors trainable."""
    from ..models.layers import FeedForward
    swapped = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, FeedForward) and not getattr(child, "glu", False):
                setattr(parent, name, BatchEnsembleFeedForward(child, n_ensembles, init))
                swapped += 1
    if freeze_shared:
        for name, p in model.named_parameters():
            p.requires_grad_(name.rsplit(".", 1)[-1] in ("r_in", "s_in", "r_out", "s_out", "r", "s"))
    return swapped
