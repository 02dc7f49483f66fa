"""Scoring utilities around a trained model: perplexity of reference translations, n-best rescoring, language
prediction, and segment-wise (streaming) translation that carries the last target tokens of the previous segment
as a forced prefix context.

Reference: onmt/inference/perplexity_scorer.py:15, onmt/Rescorer.py:14, onmt/inference/predictor.py:14,
onmt/inference/stream_translator.py:13 (the document-global beam is ``legacy_search.GlobalStreamTranslator``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

from .translator import Translator


class PerplexityScorer(Translator):
    """``score(src_sents, tgt_sents)`` -> per-sentence log-probabilities and the corpus perplexity."""

    def score(self, src_sents: List[List[str]], tgt_sents: List[List[str]], batch_size: int = 32):
        scores, words = [], 0
        for i in range(0, len(src_sents), batch_size):
            batch = self.build_data(src_sents[i:i + batch_size], tgt_sents[i:i + batch_size])
            if self.cuda:
                batch = batch.cuda(self.device)
            _, sums, _ = self.model.decode(batch)
            scores += sums.float().cpu().tolist()
            words += batch.tgt_size
        ppl = math.exp(-sum(scores) / max(words, 1))
        return scores, ppl


class Rescorer(PerplexityScorer):
    """Re-ranks n-best lists: ``rescore(src, [[hyp tokens, ...], ...])`` returns hypotheses sorted by model score
    (optionally length-normalised with ``alpha``)."""

    def rescore(self, src_sents: List[List[str]], nbest: List[List[List[str]]], alpha: float = 0.0):
        out = []
        for src, hyps in zip(src_sents, nbest):
            scores, _ = self.score([src] * len(hyps), hyps, batch_size=len(hyps))
            norm = [s / (max(len(h) + 1, 1) ** alpha) if alpha > 0 else s for s, h in zip(scores, hyps)]
            order = sorted(range(len(hyps)), key=lambda i: -norm[i])
            out.append([(hyps[i], norm[i]) for i in order])
        return out


class LanguagePredictor(Translator):
    """Predicts the language of each input from a classifier head on the encoder (models exposing ``predict_language``)."""

    def predict(self, src_sents: List[List[str]]):
        batch = self.build_data(src_sents)
        if self.cuda:
            batch = batch.cuda(self.device)
        model = self.model
        if not hasattr(model, "predict_language"):
            raise NotImplementedError("the loaded model has no language-prediction head")
        return model.predict_language(batch).argmax(-1).cpu().tolist()


class ClassifierPredictor(Translator):
    """Labels every input with a trained classifier (``-model classifier`` checkpoints: encoder + pooled linear head).
    Returns (label index, log-probability of that label) per input; ``label_name`` maps indices through the target
    dictionary.  Reference: classify.py:179-380 (batching loop, ``get_result``), onmt/inference/predictor.py."""

    def predict(self, src_sents: List[List[str]], batch_size: int = 32):
        out = []
        self.model.eval()
        for i in range(0, len(src_sents), batch_size):
            batch = self.build_data(src_sents[i:i + batch_size])
            if self.cuda:
                batch = batch.cuda(self.device)
            with torch.no_grad():
                logits = self.model(batch)["logits"].float()
            if logits.dim() == 3:                         # per-frame heads: average the frame log-probabilities
                logits = torch.log_softmax(logits, -1).mean(1)
            logp = torch.log_softmax(logits, -1)
            best = logp.argmax(-1)
            rows = list(zip(best.cpu().tolist(), logp.gather(1, best[:, None]).squeeze(1).cpu().tolist()))
            out.extend(rows)
        return out

    def label_name(self, index: int) -> str:
        d = self.tgt_dict if getattr(self, "tgt_dict", None) is not None else None
        return d.get_label(index) if d is not None and hasattr(d, "get_label") else str(index)


class StreamTranslator(Translator):
    """Translates a document segment by segment.  The tail (``context_tokens``) of the previous segment's output is
    forced as a prefix of the next hypothesis and stripped from the returned text, so lexical choices stay consistent
    across segment borders; models with segment memories (``init_stream``) also keep their hidden-state memories."""

    def __init__(self, opt, context_tokens: int = 0):
        super().__init__(opt)
        self.context_tokens = context_tokens
        self.prev: List[str] = []
        self.stream = self.model.init_stream() if hasattr(self.model, "init_stream") else None

    def reset_stream(self):
        self.prev = []
        if hasattr(self.model, "init_stream"):
            self.stream = self.model.init_stream()

    def translate_segment(self, src_tokens: List[str]) -> List[str]:
        prefix = [self.prev[-self.context_tokens:]] if (self.context_tokens and self.prev) else None
        pred, *_ = self.translate([src_tokens], prefix=prefix)
        hyp = pred[0][0]
        if prefix:
            hyp = hyp[len(prefix[0]):]
        self.prev = (self.prev + hyp)[-max(self.context_tokens, 1) * 4:]
        return hyp

