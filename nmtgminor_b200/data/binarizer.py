"""Text -> id tensors, optionally with worker processes over byte ranges of the input file.

Each worker seeks to its byte offset, realigns to the next line start, converts lines to id tensors with the
given dictionary and returns them with their sizes; results are concatenated in file order.  Counterpart of
the reference's ``Binarizer`` (onmt/data/binarizer.py:19-237) and ``Tokenizer`` (onmt/data/tokenizer.py:22-68).
"""
from __future__ import annotations

import multiprocessing as mp
import os
from typing import Callable, List, Optional, Tuple

import torch

from .. import constants as C


class Tokenizer:
    """Whitespace (word) or character tokenisation, optional lower-casing; callable on a line."""

    def __init__(self, input_type: str = "word", lower: bool = False):
        self.input_type, self.lower = input_type, lower

    def __call__(self, line: str) -> List[str]:
        line = line.strip()
        if self.lower:
            line = line.lower()
        if self.input_type == "word":
            return line.split()
        if self.input_type == "char":
            return list(line)
        raise ValueError("unknown input type %r" % self.input_type)

    tokenize = __call__


def find_offsets(path: str, n_chunks: int) -> List[int]:
    size = os.path.getsize(path)
    offs = [0]
    with open(path, "rb") as fh:
        for i in range(1, n_chunks):
            fh.seek(size * i // n_chunks)
            fh.readline()                      # move to the next line start
            offs.append(min(fh.tell(), size))
    offs.append(size)
    return offs


def binarize_range(path: str, vocab, tokenizer: Callable, start: int, end: int, bos_word: Optional[str],
                   eos_word: Optional[str], external=None) -> Tuple[List[torch.Tensor], List[int]]:
    data, sizes = [], []
    with open(path, "rb") as fh:
        fh.seek(start)
        while fh.tell() < end:
            raw = fh.readline()
            if not raw:
                break
            line = raw.decode("utf-8")
            if external is not None:
                ids = torch.tensor(external(line.strip()), dtype=torch.int64)
            else:
                ids = vocab.convert_to_idx(tokenizer(line), C.UNK_WORD, bos_word, eos_word)
            data.append(ids)
            sizes.append(int(ids.numel()))
    return data, sizes


def binarize_file(path: str, vocab, tokenizer: Optional[Callable] = None, bos_word: Optional[str] = None,
                  eos_word: Optional[str] = None, num_workers: int = 1, external=None):
    tokenizer = tokenizer or Tokenizer()
    if num_workers <= 1 or external is not None:
        data, sizes = binarize_range(path, vocab, tokenizer, 0, os.path.getsize(path), bos_word, eos_word, external)
        return {"data": data, "sizes": sizes}
    offs = find_offsets(path, num_workers)
    with mp.get_context("spawn").Pool(num_workers) as pool:
        jobs = [pool.apply_async(binarize_range, (path, vocab, tokenizer, offs[i], offs[i + 1], bos_word, eos_word))
                for i in range(num_workers)]
        parts = [j.get() for j in jobs]
    data = [t for p in parts for t in p[0]]
    sizes = [s for p in parts for s in p[1]]
    return {"data": data, "sizes": sizes}


def binarize_speech_file(path: str, fmt: str = "wav", num_mel_bin: int = 0, concat: int = 1, sample_rate: int = 16000):
    """Index an utterance list without copying the audio (reference: onmt/data/binarizer.py ``SpeechBinarizer``).

    ``fmt == "wav"``: lines ``utt_id wav_path [start end]`` (seconds) -> entries ``(wav_path, start, end, sample_rate)``;
    the size of an utterance is its number of samples (or of 10 ms feature frames when ``num_mel_bin > 0``).
    ``fmt in ("scp", "kaldi")``: lines ``utt_id ark_path:offset`` -> entries ``(ark_path, offset)``; the size is the number
    of frames after ``concat`` stacking.  Returns ``{"data": entries, "sizes": lengths}`` in file order."""
    import wave
    from .audio import read_ark_matrix
    data, sizes = [], []
    with open(path, encoding="utf-8") as fh:
        for line in fh:
            parts = line.split()
            if not parts:
                continue
            if fmt == "wav":
                wav_path = parts[1] if len(parts) > 1 else parts[0]
                start, end = (float(parts[2]), float(parts[3])) if len(parts) >= 4 else (0.0, 0.0)
                with wave.open(wav_path, "rb") as w:
                    sr, frames = w.getframerate(), w.getnframes()
                n = int(round((end - start) * sr)) if end > 0 else frames - int(round(start * sr))
                n = max(min(n, frames), 0)
                data.append((wav_path, start, end, sr))
                sizes.append(n // (sr // 100) if num_mel_bin > 0 else n)
            else:
                loc = parts[1] if len(parts) > 1 else parts[0]
                f, off = loc.rsplit(":", 1)
                rows = read_ark_matrix(f, int(off)).shape[0]
                data.append((f, int(off)))
                sizes.append((rows + concat - 1) // concat)
    return {"data": data, "sizes": sizes}


def load_external_tokenizer(name: str, lang: Optional[str] = None):
    """``-external_tokenizer <name or path>``: a Hugging Face tokenizer turns a raw line into ids (with its own special
    symbols), instead of the whitespace tokeniser + dictionary lookup.  ``name`` is a local directory or a model name that
    is present in the local cache (nothing is downloaded).  Returns ``line -> list of ids``
    (reference: onmt/data/binarizer.py, ``external_tokenizer`` branches)."""
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(name, local_files_only=True)
    if lang and hasattr(tok, "src_lang"):
        tok.src_lang = lang
    return lambda line: tok(line)["input_ids"]
