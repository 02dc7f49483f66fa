"""Hugging Face style interface for the speech-to-text models, so that scripts written against
``WhisperForConditionalGeneration`` (``model(input_features=..., labels=...) -> .loss / .logits``), and
``transformers.Seq2SeqTrainer`` where its dependencies are installed, can drive a model of this framework.

* ``HFSeq2SeqAdapter(model, pad_id, bos_id)`` - ``forward(input_features [B, n_mels, frames], labels [B, U] (-100 = ignore),
  attention_mask=None)`` builds the packed batch this framework's models take (frames as rows, labels shifted right
  behind ``bos_id`` as decoder input), returns a ``Seq2SeqOutput`` with ``loss`` (mean over the labelled tokens, as the
  Hugging Face models report it) and, with ``return_logits=True``, ``logits [B, U, V]``.
* ``SpeechSeq2SeqCollator`` - list of ``{"input_features": [n_mels, frames], "labels": [U]}`` -> padded batch dictionary
  (what ``DataCollatorSpeechSeq2SeqWithPadding`` of the Whisper fine-tuning recipes produces).
* ``train_steps`` - a plain loop (AdamW, gradient clipping) for environments without ``accelerate``, which
  ``transformers.Trainer`` needs; ``make_trainer`` builds a ``Seq2SeqTrainer`` when that import works.

Reference: whisper/train_whisper.py:430-640 (collator, trainer construction, training arguments),
whisper/memory_efficient_whisper.py:237-330 (``forward`` with labels and the fused cross-entropy).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..data.dataset import collate

IGNORE = -100


@dataclass
class Seq2SeqOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    n_tokens: int = 0

    def __getitem__(self, k):          # tuple / dict style access used by the trainer's prediction step
        return (self.loss, self.logits)[k] if isinstance(k, int) else getattr(self, k)


class HFSeq2SeqAdapter(nn.Module):
    def __init__(self, model: nn.Module, pad_id: int = 0, bos_id: int = 2):
        super().__init__()
        self.model, self.pad_id, self.bos_id = model, pad_id, bos_id
        self.config = getattr(model, "opt", None)

    def _batch(self, input_features, labels, attention_mask):
        B = input_features.shape[0]
        feats = input_features.transpose(1, 2)                                     # [B, frames, n_mels]
        if attention_mask is not None:
            lengths = attention_mask.sum(-1).tolist()
        else:
            lengths = [feats.shape[1]] * B
        src = [feats[i, :int(lengths[i])].float().cpu() for i in range(B)]
        tgt = []
        for i in range(B):
            y = labels[i][labels[i] != IGNORE].cpu()
            tgt.append(torch.cat([torch.tensor([self.bos_id], dtype=torch.long), y.long()]))   # decoder input | labels are its shift
        return collate(src, tgt, src_type="audio", padded=True, packed=True, round_to=16)

    def forward(self, input_features=None, labels=None, attention_mask=None, return_logits: bool = False, **_unused):
        batch = self._batch(input_features, labels, attention_mask)
        dev = next(self.model.parameters()).device
        if dev.type == "cuda":
            batch = batch.cuda(dev)
        out = self.model(batch, return_logits=return_logits)
        n = int(batch.tgt_size)
        loss = out["loss"].sum() / max(n, 1)
        logits = None
        if return_logits:
            logits = out["logprobs"].transpose(0, 1)                                # [B, U, V]
        return Seq2SeqOutput(loss=loss, logits=logits, n_tokens=n)


class SpeechSeq2SeqCollator:
    """Pads ``input_features`` with zeros (and reports an ``attention_mask`` over frames) and ``labels`` with -100."""

    def __call__(self, features: List[Dict]) -> Dict[str, torch.Tensor]:
        F = max(f["input_features"].shape[-1] for f in features)
        U = max(len(f["labels"]) for f in features)
        x = torch.zeros(len(features), features[0]["input_features"].shape[0], F)
        mask = torch.zeros(len(features), F, dtype=torch.long)
        y = torch.full((len(features), U), IGNORE, dtype=torch.long)
        for i, f in enumerate(features):
            n = f["input_features"].shape[-1]
            x[i, :, :n] = torch.as_tensor(f["input_features"])
            mask[i, :n] = 1
            y[i, :len(f["labels"])] = torch.as_tensor(f["labels"])
        return {"input_features": x, "attention_mask": mask, "labels": y}


def train_steps(adapter: HFSeq2SeqAdapter, batches, lr: float = 1e-5, weight_decay: float = 0.01, max_grad_norm: float = 1.0,
                optimizer: Optional[torch.optim.Optimizer] = None) -> List[float]:
    """One AdamW update per batch dictionary; returns the losses (what ``Seq2SeqTrainer`` logs as ``loss``)."""
    params = [p for p in adapter.parameters() if p.requires_grad]
    opt = optimizer or torch.optim.AdamW(params, lr=lr, weight_decay=weight_decay)
    adapter.train()
    losses = []
    for b in batches:
        out = adapter(**b)
        out.loss.backward()
        torch.nn.utils.clip_grad_norm_(params, max_grad_norm)
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(out.loss.detach()))
    return losses


def make_trainer(adapter: HFSeq2SeqAdapter, train_dataset, eval_dataset=None, **training_args):
    """``transformers.Seq2SeqTrainer`` around the adapter (full-shard FSDP, schedulers and callbacks are then the
    trainer's).  Raises ``ImportError`` with the missing package's name when the trainer cannot be constructed."""
    try:
        import accelerate  # noqa: F401  (transformers.Trainer refuses to start without it)
        from transformers import Seq2SeqTrainer, Seq2SeqTrainingArguments
    except ImportError as exc:
        raise ImportError("transformers.Seq2SeqTrainer needs %s; use train_steps() or this framework's trainer "
                          "(finetune_whisper.py) instead" % (exc.name or "accelerate")) from exc
    args = Seq2SeqTrainingArguments(remove_unused_columns=False, **training_args)
    return Seq2SeqTrainer(model=adapter, args=args, train_dataset=train_dataset, eval_dataset=eval_dataset,
                          data_collator=SpeechSeq2SeqCollator())
