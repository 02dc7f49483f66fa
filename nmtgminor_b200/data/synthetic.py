"""Synthetic corpora of the benchmark shapes (no data set can be downloaded where this runs).

Token ids are uniform over the non-special vocabulary, lengths uniform in a range; targets are wrapped in
BOS ... EOS.  ``make_static_batches`` additionally pads every batch to the same packed capacities so the
training step can be captured in a CUDA graph.
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np
import torch

from .. import constants as C
from ..dictionary import Dict
from .dataset import Batch, Dataset, collate


def synthetic_dict(vocab_size: int) -> Dict:
    d = Dict([C.PAD_WORD, C.UNK_WORD, C.BOS_WORD, C.EOS_WORD])
    for i in range(vocab_size - 4):
        d.add("w%d" % i)
    return d


def synthetic_pairs(n: int, vocab: int, min_len: int, max_len: int, seed: int = 1) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    """n sentence pairs; source = plain ids, target = BOS ids EOS; lengths count content tokens."""
    rng = np.random.RandomState(seed)
    src, tgt = [], []
    for _ in range(n):
        ls, lt = rng.randint(min_len, max_len + 1), rng.randint(min_len, max_len + 1)
        src.append(torch.from_numpy(rng.randint(4, vocab, size=ls).astype(np.int64)))
        body = rng.randint(4, vocab, size=lt).astype(np.int64)
        tgt.append(torch.from_numpy(np.concatenate([[C.BOS], body, [C.EOS]]).astype(np.int64)))
    return src, tgt


def synthetic_dataset(n: int, vocab: int, min_len: int, max_len: int, batch_size_words: int, seed: int = 1, **kw) -> Dataset:
    src, tgt = synthetic_pairs(n, vocab, min_len, max_len, seed)
    return Dataset(src, tgt, batch_size_words=batch_size_words, max_src_len=max_len + 3, max_tgt_len=max_len + 3, **kw)


def token_budget_batches(vocab: int, min_len: int, max_len: int, tokens_per_batch: int, n_batches: int, seed: int = 1,
                         static: bool = True, round_to: int = 128, padded: bool = False) -> List[Batch]:
    """Batches holding ~``tokens_per_batch`` TARGET tokens each (sum of real lengths, no padding waste)."""
    rng = np.random.RandomState(seed)
    groups = []
    for _ in range(n_batches):
        src, tgt, tot = [], [], 0
        while True:
            ls, lt = rng.randint(min_len, max_len + 1), rng.randint(min_len, max_len + 1)
            if tot + lt + 1 > tokens_per_batch and tgt:
                break
            src.append(torch.from_numpy(rng.randint(4, vocab, size=ls).astype(np.int64)))
            body = rng.randint(4, vocab, size=lt).astype(np.int64)
            tgt.append(torch.from_numpy(np.concatenate([[C.BOS], body, [C.EOS]]).astype(np.int64)))
            tot += lt + 1
        groups.append((src, tgt))
    cap_s = cap_t = max_b = None
    if static:
        up = lambda v: (v + round_to - 1) // round_to * round_to
        cap_s = up(max(sum(len(s) for s in g[0]) for g in groups))
        cap_t = up(max(sum(len(t) - 1 for t in g[1]) for g in groups))
        max_b = max(len(g[0]) for g in groups)
    out = []
    for src, tgt in groups:
        out.append(collate(src, tgt, padded=padded, packed=True, capacity_src=cap_s, capacity_tgt=cap_t, max_batch=max_b,
                           round_to=round_to))
    if static:
        # a common upper bound on sequence length keeps attention grids identical across batches
        m_s = max(b.packed_source().max_len for b in out)
        m_t = max(b.packed_target_input().max_len for b in out)
        for b in out:
            b.packed_source().max_len = m_s
            b.packed_target_input().max_len = m_t
    return out


def synthetic_audio_batch(n: int, vocab: int, kind: str = "wav", min_len: int = 4000, max_len: int = 8000, n_feats: int = 80,
                          tgt_min: int = 5, tgt_max: int = 20, seed: int = 1, fixed_frames: int = 0) -> Batch:
    """Speech batch: raw 16 kHz waveforms ~N(0, 0.1) (``kind='wav'``) or feature matrices ~N(0, 1) (``kind='feats'``:
    log-mel / filterbank frames; ``fixed_frames`` > 0 gives every utterance that many frames, as Whisper's 30 s windows)."""
    rng = np.random.RandomState(seed)
    src, tgt = [], []
    for _ in range(n):
        L = fixed_frames if fixed_frames > 0 else int(rng.randint(min_len, max_len + 1))
        if kind == "wav":
            src.append(torch.from_numpy((rng.randn(L, 1) * 0.1).astype(np.float32)))
        else:
            src.append(torch.from_numpy(rng.randn(L, n_feats).astype(np.float32)))
        lt = int(rng.randint(tgt_min, tgt_max + 1))
        tgt.append(torch.from_numpy(np.concatenate([[C.BOS], rng.randint(4, vocab, size=lt), [C.EOS]]).astype(np.int64)))
    return collate(src, tgt, src_type="audio", padded=True, packed=True, round_to=16)
