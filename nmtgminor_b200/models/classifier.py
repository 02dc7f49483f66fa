"""Sequence classifier on top of any encoder of the framework (``train_classify.py`` / ``classify.py``): encoder states are
mean-pooled (``-classifier_pooling mean``) or classified per frame, then projected to the label set.
Reference: onmt/model_factory.py:68 (``build_classifier``), onmt/models/speech_recognizer/classifier.py, onmt/train_utils/classify_trainer.py:73.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Embedding
from .transformer import TransformerEncoder


class Classifier(nn.Module):
    def __init__(self, opt, dicts):
        super().__init__()
        self.opt = opt
        n_labels = dicts["tgt"].size() if "tgt" in dicts else getattr(opt, "n_classes", 2)
        if getattr(opt, "encoder_type", "text") == "text":
            self.encoder = TransformerEncoder(opt, Embedding(dicts["src"].size(), opt.model_size, getattr(opt, "pad_idx", 0)))
            self.speech = False
        else:
            name = (getattr(opt, "enc_pretrained_model", "") or "").lower()
            if "wav2vec" in name or "hubert" in name or "wavlm" in name:
                from .pretrained import _wav2vec_from_opt
                self.encoder = _wav2vec_from_opt(opt)
            else:
                from .speech_encoders import SpeechTransformerEncoder
                self.encoder = SpeechTransformerEncoder(opt, getattr(opt, "input_size", 40))
            self.speech = True
        self.head = nn.Linear(self.encoder.dim if hasattr(self.encoder, "dim") else opt.model_size, n_labels)
        self.pooling = getattr(opt, "classifier_pooling", "mean")

    def forward(self, batch, **_unused):
        if self.speech:
            states, seqs = self.encoder(batch.get("source"))
        else:
            seqs = batch.packed_source()
            states = self.encoder(seqs)
        padded = seqs.pad(states.float(), time_first=False)               # [B, T, H]
        lengths = (seqs.cu[1:] - seqs.cu[:-1]).clamp(min=1)
        if self.pooling == "mean":
            pooled = padded.sum(1) / lengths[:, None]
            logits = self.head(pooled)
        else:
            logits = self.head(padded)
        out = {"logits": logits, "src": seqs}
        labels = batch.get("labels")
        if labels is not None and logits.dim() == 2:
            out["loss"] = F.cross_entropy(logits, labels.to(logits.device), reduction="sum")
            out["correct"] = (logits.argmax(-1) == labels.to(logits.device)).sum().float().reshape(1)
        return out


def register_builders(register):
    register("classifier")(lambda opt, dicts: Classifier(opt, dicts))
