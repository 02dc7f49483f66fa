"""Vocabulary: word <-> id map with special tokens, frequency pruning and size padding.

Same role and on-disk content (``idxToLabel``, ``labelToIdx``, ``frequencies``, ``special``) as the
reference's ``onmt.Dict`` (onmt/Dict.py:10-289), so a dictionary pickled by either side can be read by
the other through ``Dict.from_state`` / ``state``.
"""
from __future__ import annotations

from collections import Counter
from typing import Iterable, List, Optional

import torch

from . import constants as C


class Dict:
    def __init__(self, data=None, lower: bool = False):
        self.idxToLabel = {}
        self.labelToIdx = {}
        self.frequencies = {}
        self.lower = lower
        self.special: List[int] = []
        if data is not None:
            if isinstance(data, str):
                self.load_file(data)
            else:
                self.add_specials(data)

    # -- basic -------------------------------------------------------------------------------------
    def size(self) -> int:
        return len(self.idxToLabel)

    __len__ = size

    def load_file(self, path: str) -> None:
        with open(path, encoding="utf-8") as fh:
            for line in fh:
                fields = line.rstrip("\n").split()
                if not fields:
                    continue
                if len(fields) >= 2 and fields[-1].lstrip("-").isdigit():
                    label, idx = " ".join(fields[:-1]), int(fields[-1])
                    self.add(label, idx)
                else:
                    self.add(fields[0])

    def write_file(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as fh:
            for i in range(self.size()):
                fh.write("%s %d\n" % (self.idxToLabel[i], i))

    def lookup(self, key: str, default=None):
        key = key.lower() if self.lower else key
        return self.labelToIdx.get(key, default)

    def get_label(self, idx: int, default=None):
        return self.idxToLabel.get(idx, default)

    getLabel = get_label

    def add_special(self, label: str, idx: Optional[int] = None) -> None:
        self.special.append(self.add(label, idx))

    def add_specials(self, labels: Iterable[str]) -> None:
        for label in labels:
            self.add_special(label)

    addSpecial, addSpecials = add_special, add_specials

    def add(self, label: str, idx: Optional[int] = None, num: int = 1) -> int:
        label = label.lower() if self.lower else label
        if idx is not None:
            self.idxToLabel[idx] = label
            self.labelToIdx[label] = idx
        elif label in self.labelToIdx:
            idx = self.labelToIdx[label]
        else:
            idx = len(self.idxToLabel)
            self.idxToLabel[idx] = label
            self.labelToIdx[label] = idx
        self.frequencies[idx] = self.frequencies.get(idx, 0) + num
        return idx

    # -- vocabulary shaping ------------------------------------------------------------------------
    def prune(self, size: int) -> "Dict":
        """Keep the specials plus the ``size`` most frequent words."""
        if size >= self.size():
            return self
        order = sorted((i for i in self.frequencies if i not in self.special), key=lambda i: -self.frequencies[i])
        out = Dict(lower=self.lower)
        for i in self.special:
            out.add_special(self.idxToLabel[i])
        for i in order[:size]:
            out.add(self.idxToLabel[i], num=self.frequencies[i])
        return out

    def patch(self, multiplier: int = 8) -> None:
        """Pad the vocabulary with dummy words so its size is a multiple of ``multiplier`` (tensor-core friendly)."""
        n = 0
        while self.size() % multiplier:
            self.add("<extra_%d>" % n)
            n += 1

    # -- conversion --------------------------------------------------------------------------------
    def convert_to_idx(self, labels, unk_word=C.UNK_WORD, bos_word=None, eos_word=None, type="int64"):
        vec = []
        if bos_word is not None:
            vec.append(self.lookup(bos_word))
        unk = self.lookup(unk_word)
        vec.extend(self.lookup(w, unk) for w in labels)
        if eos_word is not None:
            vec.append(self.lookup(eos_word))
        return torch.tensor(vec, dtype=torch.int64 if type == "int64" else torch.int32)

    def convert_to_labels(self, idx, stop=None, including_stop=True) -> List[str]:
        out = []
        for i in idx:
            i = int(i)
            if stop is not None and i == stop and not including_stop:
                break
            out.append(self.get_label(i, C.UNK_WORD))
            if stop is not None and i == stop:
                break
        return out

    convertToIdx, convertToLabels = convert_to_idx, convert_to_labels

    # -- construction from corpora -----------------------------------------------------------------
    @staticmethod
    def count_file(path: str, tokenizer=str.split, lower=False) -> Counter:
        c = Counter()
        with open(path, encoding="utf-8") as fh:
            for line in fh:
                toks = tokenizer(line.strip())
                c.update(t.lower() for t in toks) if lower else c.update(toks)
        return c

    @staticmethod
    def build(counters: Iterable[Counter], size: int = 0, specials=(C.PAD_WORD, C.UNK_WORD, C.BOS_WORD, C.EOS_WORD),
              lower=False) -> "Dict":
        total = Counter()
        for c in counters:
            total.update(c)
        d = Dict(list(specials), lower=lower)
        for w, n in sorted(total.items(), key=lambda kv: (-kv[1], kv[0])):
            d.add(w, num=n)
        return d.prune(size) if size and size < d.size() else d

    # -- (de)serialisation in the reference's attribute layout --------------------------------------
    def state(self) -> dict:
        return {"idxToLabel": self.idxToLabel, "labelToIdx": self.labelToIdx, "frequencies": self.frequencies,
                "lower": self.lower, "special": self.special}

    @staticmethod
    def from_state(obj) -> "Dict":
        st = obj if isinstance(obj, dict) else vars(obj)
        d = Dict(lower=st.get("lower", False))
        d.idxToLabel = dict(st["idxToLabel"])
        d.labelToIdx = dict(st["labelToIdx"])
        d.frequencies = dict(st.get("frequencies", {}))
        d.special = list(st.get("special", []))
        return d
