"""Text utilities: vocabulary extraction, text normalisation, sampling from a language model, and an auto-encoder
over encoder states.

Reference: extract_vocab.py, normalize_text.py, sample_lm.py, autoencoder.py / eval_autoencoder.py / ae/ (Autoencoder,
AETrainer).
"""
from __future__ import annotations

import re
import unicodedata
from collections import Counter
from typing import Iterable, List

import torch
import torch.nn as nn


def extract_vocab(lines: Iterable[str], min_count: int = 1, max_size: int = 0, lower: bool = False) -> List[str]:
    c = Counter()
    for line in lines:
        c.update((line.lower() if lower else line).split())
    words = [w for w, n in sorted(c.items(), key=lambda kv: (-kv[1], kv[0])) if n >= min_count]
    return words[:max_size] if max_size else words


_PUNCT = re.compile(r"\s+([?.!,;:])")


def normalize_text(line: str, lower: bool = False, strip_punct: bool = False) -> str:
    line = unicodedata.normalize("NFKC", line)
    line = re.sub(r"[‘’]", "'", line)
    line = re.sub(r"[“”]", '"', line)
    line = re.sub(r"\s+", " ", line).strip()
    if strip_punct:
        line = "".join(ch for ch in line if not unicodedata.category(ch).startswith("P") or ch == "'")
        line = re.sub(r"\s+", " ", line).strip()
    return line.lower() if lower else line


@torch.no_grad()
def sample_lm(model, dictionary, prefix: List[str], max_len: int = 50, temperature: float = 1.0, top_k: int = 0, seed: int = 0):
    """Ancestral sampling from a decoder-only language model exposing ``logits(tokens [B, T]) -> [B, T, V]`` or the
    framework's ``forward(batch)`` with ``return_logits``."""
    from ..data.dataset import collate
    g = torch.Generator().manual_seed(seed)
    ids = dictionary.convert_to_idx(prefix, "<unk>", "<s>").tolist()
    for _ in range(max_len):
        row = torch.tensor(ids + [0])
        batch = collate(None, [row], round_to=1)
        out = model(batch, return_logits=True, compute_loss=False)
        logits = out["logprobs"][len(ids) - 1, 0].float() / max(temperature, 1e-5)
        if top_k > 0:
            kth = logits.topk(top_k).values[-1]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        nxt = int(torch.multinomial(torch.softmax(logits, -1), 1, generator=g))
        ids.append(nxt)
        if nxt == 3:
            break
    return dictionary.convert_to_labels(ids[1:], 3, including_stop=False)


class Autoencoder(nn.Module):
    """Bottleneck auto-encoder over hidden states of a trained model (``hidden -> inner -> hidden``)."""

    def __init__(self, input_size: int, inner_size: int = 256, layers: int = 1, dropout: float = 0.0):
        super().__init__()
        dims = [input_size] + [inner_size] * layers
        enc, dec = [], []
        for a, b in zip(dims[:-1], dims[1:]):
            enc += [nn.Linear(a, b), nn.Tanh(), nn.Dropout(dropout)]
        for a, b in zip(reversed(dims[1:]), reversed(dims[:-1])):
            dec += [nn.Linear(a, b), nn.Tanh()]
        self.encoder, self.decoder = nn.Sequential(*enc), nn.Sequential(*dec[:-1])

    def forward(self, x):
        return self.decoder(self.encoder(x))

    def loss(self, x, mask=None):
        err = (self.forward(x) - x) ** 2
        if mask is not None:
            err = err * mask[..., None]
            return err.sum() / mask.sum().clamp_min(1) / x.shape[-1]
        return err.mean()


def train_autoencoder(states: List[torch.Tensor], inner_size: int = 64, epochs: int = 5, lr: float = 1e-3, seed: int = 0) -> Autoencoder:
    torch.manual_seed(seed)
    ae = Autoencoder(states[0].shape[-1], inner_size)
    opt = torch.optim.Adam(ae.parameters(), lr=lr)
    for _ in range(epochs):
        for s in states:
            opt.zero_grad()
            ae.loss(s).backward()
            opt.step()
    return ae
