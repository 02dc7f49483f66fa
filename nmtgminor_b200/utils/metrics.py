"""Corpus / sentence BLEU, GLEU and hit rate on token lists.  Counterparts of onmt/metrics/{bleu,sbleu,gleu,hit}.py."""
from __future__ import annotations

import math
from collections import Counter
from typing import List, Sequence


def _ngrams(tokens: Sequence, n: int) -> Counter:
    return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


def bleu_stats(hyp: Sequence, ref: Sequence, max_n: int = 4):
    stats = [len(hyp), len(ref)]
    for n in range(1, max_n + 1):
        h, r = _ngrams(hyp, n), _ngrams(ref, n)
        stats += [sum((h & r).values()), max(len(hyp) - n + 1, 0)]
    return stats


def bleu_from_stats(stats, smooth: float = 0.0) -> float:
    c, r = stats[0], stats[1]
    if c == 0:
        return 0.0
    logp = 0.0
    n = (len(stats) - 2) // 2
    for i in range(n):
        m, t = stats[2 + 2 * i] + smooth, stats[3 + 2 * i] + smooth
        if m <= 0 or t <= 0:
            return 0.0
        logp += math.log(m / t) / n
    bp = min(0.0, 1.0 - r / c)
    return 100.0 * math.exp(logp + bp)


def corpus_bleu(hyps: List[Sequence], refs: List[Sequence], max_n: int = 4) -> float:
    total = [0] * (2 + 2 * max_n)
    for h, r in zip(hyps, refs):
        total = [a + b for a, b in zip(total, bleu_stats(h, r, max_n))]
    return bleu_from_stats(total)


def sentence_bleu(hyp: Sequence, ref: Sequence, max_n: int = 4) -> float:
    """Add-one smoothed sentence-level BLEU."""
    return bleu_from_stats(bleu_stats(hyp, ref, max_n), smooth=1.0) if len(hyp) else 0.0


def sentence_gleu(hyp: Sequence, ref: Sequence, max_n: int = 4) -> float:
    match = total_h = total_r = 0
    for n in range(1, max_n + 1):
        h, r = _ngrams(hyp, n), _ngrams(ref, n)
        match += sum((h & r).values())
        total_h += sum(h.values())
        total_r += sum(r.values())
    denom = max(total_h, total_r)
    return match / denom if denom else 0.0


def hit_rate(hyp: Sequence, ref: Sequence) -> float:
    if not ref:
        return 0.0
    rs = set(ref)
    return sum(1 for t in set(hyp) if t in rs) / len(rs)
