"""Datasets, bucketed batching and the ``Batch`` object consumed by models.

``Dataset`` holds per-sentence tensors (token ids, or ``[frames, features]`` matrices for speech), filters
them by length, sorts them by size, and cuts token-budget batches with the C++ allocator
(``ops/csrc/batch_alloc.cpp``; a Python restatement is used when the extension is absent).  ``collate``
produces a ``Batch`` whose tensors use the reference's key names and ``[T, B]`` layout
(onmt/data/dataset.py:360-541 ``collate_fn``, :604-678 ``Batch``) and which additionally offers *packed*
views (``packed_source`` / ``packed_target_input`` / ``packed_target_output``): concatenated tokens plus
cumulative lengths, the layout every kernel of this framework works on.  Packing happens on the host in
``collate`` so the per-step host-to-device traffic is a handful of small integer tensors.

Reference behaviour: onmt/data/dataset.py:707-1344 ``Dataset``, onmt/data/batch_utils.py:7-286.
"""
from __future__ import annotations

import math
from typing import Dict as TDict, List, Optional, Sequence

import numpy as np
import torch

from .. import constants as C
from ..models.layers import PackedSeqs


# ---------------------------------------------------------------------------------------------------
# batch allocation
# ---------------------------------------------------------------------------------------------------
def allocate_batches_python(indices, lengths, src_sizes, tgt_sizes, batch_size_words, batch_size_frames, batch_size_sents,
                            multiplier, max_src_len, max_tgt_len, min_src_len, min_tgt_len, cleaning=True,
                            unbalanced=False, cut_off_size=256000, smallest_batch_size=4) -> List[List[int]]:
    """Readable restatement of the C++ allocator (also its test oracle)."""
    batches, cur, words, frames = [], [], [], []
    multiplier = max(1, multiplier)
    for i in indices:
        src = src_sizes[i] if src_sizes is not None else (min_src_len if unbalanced else 0)
        tgt = tgt_sizes[i] if tgt_sizes is not None else (min_tgt_len if unbalanced else 0)
        if cleaning and not (min_src_len <= src < max_src_len and min_tgt_len <= tgt < max_tgt_len):
            continue
        nw = tgt if unbalanced else lengths[i]
        nf = src
        over = False
        if cur:
            if len(cur) >= batch_size_sents:
                over = True
            elif unbalanced:
                f = max(max(frames), nf)
                if f > cut_off_size and len(cur) >= smallest_batch_size:
                    over = True
                elif f * (len(cur) + 1) > batch_size_frames:
                    over = True
                elif max(max(words), nw) * (len(cur) + 1) > batch_size_words:
                    over = True
            elif max(max(words), nw) * (len(cur) + 1) > batch_size_words:
                over = True
        if over:
            keep = max(multiplier * (len(cur) // multiplier), len(cur) % multiplier)
            batches.append(cur[:keep])
            cur, words, frames = cur[keep:], words[keep:], frames[keep:]
        cur.append(int(i))
        words.append(nw)
        frames.append(nf)
    if cur:
        batches.append(cur)
    return batches


def allocate_batches(indices, lengths, src_sizes, tgt_sizes, batch_size_words, batch_size_frames=10 ** 12,
                     batch_size_sents=10 ** 9, multiplier=1, max_src_len=10 ** 9, max_tgt_len=10 ** 9, min_src_len=0,
                     min_tgt_len=0, cleaning=True, unbalanced=False, cut_off_size=256000, smallest_batch_size=4):
    from .. import ops
    ext = ops.load_extension(build_if_missing=False)
    to_t = lambda a: None if a is None else torch.as_tensor(np.asarray(a), dtype=torch.int64)
    if ext is not None and hasattr(ext, "batch_allocate"):
        flat, offs = ext.batch_allocate(to_t(indices), to_t(lengths), to_t(src_sizes), to_t(tgt_sizes), int(batch_size_words),
                                        int(batch_size_frames), int(batch_size_sents), int(multiplier), int(max_src_len),
                                        int(max_tgt_len), int(min_src_len), int(min_tgt_len), bool(cleaning), bool(unbalanced),
                                        int(cut_off_size), int(smallest_batch_size))
        flat, offs = flat.tolist(), offs.tolist()
        return [flat[offs[i]:offs[i + 1]] for i in range(len(offs) - 1)]
    return allocate_batches_python(list(indices), lengths, src_sizes, tgt_sizes, batch_size_words, batch_size_frames,
                                   batch_size_sents, multiplier, max_src_len, max_tgt_len, min_src_len, min_tgt_len,
                                   cleaning, unbalanced, cut_off_size, smallest_batch_size)


# ---------------------------------------------------------------------------------------------------
# Batch
# ---------------------------------------------------------------------------------------------------
def _pad_stack(seqs: Sequence[torch.Tensor], pad: int):
    """List of 1-D (text) or 2-D (frames x feat) tensors -> right-padded [B, T(, 1+F)] + lengths."""
    lengths = [int(s.shape[0]) for s in seqs]
    T = max(lengths) if lengths else 0
    if seqs and seqs[0].dim() == 2:
        F = seqs[0].shape[1]
        out = torch.zeros(len(seqs), T, F + 1, dtype=seqs[0].dtype if seqs[0].is_floating_point() else torch.float32)
        for i, s in enumerate(seqs):
            out[i, :lengths[i], 1:] = s
            out[i, :lengths[i], 0] = 1          # channel 0 flags real frames (0 = padding)
        return out, lengths
    out = torch.full((len(seqs), T), pad, dtype=torch.int64)
    for i, s in enumerate(seqs):
        out[i, :lengths[i]] = s
    return out, lengths


class Batch:
    """Dictionary of batch tensors with the reference's key names plus packed views."""

    def __init__(self, tensors: TDict):
        self.tensors = tensors
        self.size = tensors.get("size", 0)
        self.src_size = tensors.get("src_size", 0)
        self.tgt_size = tensors.get("tgt_size", 0)
        self.has_target = tensors.get("target") is not None
        self._packed: TDict[str, PackedSeqs] = {k: v for k, v in tensors.items() if isinstance(v, PackedSeqs)}

    def get(self, name, default=None):
        return self.tensors.get(name, default)

    def __contains__(self, name):
        return name in self.tensors

    # packed accessors ---------------------------------------------------------------------------
    def packed_source(self) -> PackedSeqs:
        return self._packed["packed_source"]

    def packed_target_input(self) -> PackedSeqs:
        return self._packed["packed_target_input"]

    def packed_target_output(self) -> torch.Tensor:
        return self.tensors["packed_target_output"]

    # device movement ----------------------------------------------------------------------------
    def pin_memory(self):
        for k, v in list(self.tensors.items()):
            if isinstance(v, torch.Tensor):
                self.tensors[k] = v.pin_memory()
            elif isinstance(v, PackedSeqs):
                pinned = PackedSeqs(v.tokens.pin_memory(), v.positions.pin_memory(), v.cu.pin_memory(), v.max_len,
                                    v.lengths.pin_memory() if v.lengths is not None else None, v.extras)
                self.tensors[k] = pinned
                self._packed[k] = pinned
        return self

    def h2d_bytes(self, hot_only: bool = True) -> int:
        """Bytes that ``cuda(hot_only=...)`` copies to the device."""
        n = 0
        for k, v in self.tensors.items():
            if isinstance(v, PackedSeqs):
                n += v.tokens.numel() * 8 + v.positions.numel() * 8 + v.cu.numel() * 4
            elif isinstance(v, torch.Tensor) and (not hot_only or k == "packed_target_output"
                                                  or self.tensors.get("src_type", "text") != "text"):
                n += v.numel() * v.element_size()
        return n

    def cuda(self, device=None, fp16: bool = False, hot_only: bool = False, non_blocking: bool = True):
        """Move tensors to the device.  ``hot_only`` moves just what the packed training step reads."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        for k, v in list(self.tensors.items()):
            if isinstance(v, PackedSeqs):
                moved = v.to(dev, non_blocking)
                self.tensors[k] = moved
                self._packed[k] = moved
            elif isinstance(v, torch.Tensor):
                # text batches: the packed views are all the training step reads; audio batches are read through
                # their padded tensors (frames, lengths, CTC labels), so everything moves
                if hot_only and k != "packed_target_output" and self.tensors.get("src_type", "text") == "text":
                    continue
                t = v.to(dev, non_blocking=non_blocking)
                if fp16 and t.is_floating_point():
                    t = t.to(torch.bfloat16)
                self.tensors[k] = t
        return self

    to = cuda


def pack_sequences(seqs: Sequence[torch.Tensor], pad: int, capacity: Optional[int] = None, round_to: int = 1) -> PackedSeqs:
    """Concatenate 1-D token tensors; rows past the last sequence hold ``pad`` (capacity rounding)."""
    lengths = torch.tensor([int(s.shape[0]) for s in seqs], dtype=torch.int64)
    total = int(lengths.sum()) if len(seqs) else 0
    cap = capacity if capacity is not None else (total + round_to - 1) // round_to * round_to
    assert cap >= total, "packed capacity %d is below the token count %d" % (cap, total)
    toks = torch.full((cap,), pad, dtype=torch.int64)
    pos = torch.zeros((cap,), dtype=torch.int64)
    if total:
        toks[:total] = torch.cat(list(seqs))
        pos[:total] = torch.cat([torch.arange(int(n)) for n in lengths.tolist()])
    cu = torch.zeros(len(seqs) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lengths, 0).to(torch.int32)
    return PackedSeqs(toks, pos, cu, int(lengths.max()) if len(seqs) else 0, lengths)


def bucket_capacity(n: int, per_octave: int = 8, floor: int = 128) -> int:
    """Round a packed token count up to one of ``per_octave`` sizes per power of two (at most 1 / per_octave of the
    rows are padding).  Batches whose rounded sizes agree share one captured CUDA graph of the training step."""
    n = max(int(n), 1)
    if n <= floor:
        return floor
    step = max(floor, 1 << max(0, n.bit_length() - 1 - max(per_octave.bit_length() - 1, 0)))
    return (n + step - 1) // step * step


def bucket_max_len(n: int) -> int:
    """Upper bound on the sequence length that the attention kernels size their grids with: 128 (the single-tile
    kernels) or the next multiple of 128."""
    return 128 if n <= 128 else (n + 127) // 128 * 128


def collate(src_data, tgt_data, src_lang=None, tgt_lang=None, src_atb=None, tgt_atb=None, src_pad=C.PAD, tgt_pad=C.PAD,
            src_type="text", index_data=None, padded: bool = True, packed: bool = True, capacity_src: Optional[int] = None,
            capacity_tgt: Optional[int] = None, max_batch: Optional[int] = None, round_to: int = 128,
            create_reverse: bool = False, vocab_mask=None, past_src_data=None, aux_tgt_data=None,
            static_shapes: bool = False) -> Batch:
    """Build a ``Batch`` from lists of per-sentence tensors (targets carry BOS ... EOS).  ``past_src_data``: the previous
    source sentence of every example (document-context models; keys ``past_source*`` of the reference's batches).
    ``aux_tgt_data``: a second target per example ("triangle" corpora: e.g. the transcript next to the translation),
    given as ``aux_target_input`` / ``aux_target_output`` ``[T, B]`` and ``aux_tgt_lengths``.
    ``static_shapes``: round the packed capacities, the sentence count and the length bounds to a small set of sizes
    (``bucket_capacity``), so that the batches of a token-budget data set fall into a handful of shape classes."""
    if static_shapes and packed and src_type == "text":
        n_sent = len(src_data) if src_data is not None else len(tgt_data)
        if capacity_src is None and src_data is not None:
            capacity_src = bucket_capacity(sum(int(s.shape[0]) for s in src_data))
        if capacity_tgt is None and tgt_data is not None:
            capacity_tgt = bucket_capacity(sum(int(s.shape[0]) - 1 for s in tgt_data))
        if max_batch is None:
            max_batch = bucket_capacity(n_sent, per_octave=4, floor=8)
    t: TDict = {"src_type": src_type, "vocab_mask": vocab_mask}
    if aux_tgt_data is not None:
        aux_bt, aux_lengths = _pad_stack(aux_tgt_data, tgt_pad)
        t["aux_target_input"] = aux_bt[:, :-1].t().contiguous()
        t["aux_target_output"] = aux_bt[:, 1:].t().contiguous()
        t["aux_tgt_lengths"] = torch.tensor([l - 1 for l in aux_lengths], dtype=torch.int64)
    if past_src_data is not None and src_type == "text":
        past_bt, past_lengths = _pad_stack(past_src_data, src_pad)
        t["past_source"] = past_bt.t().contiguous()
        t["past_src_lengths"] = torch.tensor(past_lengths, dtype=torch.int64)
        t["past_src_selfattn_mask"] = past_bt.eq(src_pad)
        if packed:
            t["packed_past_source"] = pack_sequences(past_src_data, src_pad, None, round_to)
    if src_data is not None:
        if padded or src_type != "text":
            src_bt, src_lengths = _pad_stack(src_data, src_pad)
            if src_type == "text":
                t["src_selfattn_mask"] = src_bt.eq(src_pad)
                t["source"] = src_bt.t().contiguous()
                t["source_pos"] = torch.arange(src_bt.shape[1])[:, None].expand(-1, len(src_data)).contiguous()
            else:
                t["src_selfattn_mask"] = src_bt[:, :, 0].eq(0)
                t["source"] = src_bt.transpose(0, 1).contiguous()
                t["source_pos"] = None
        else:
            src_lengths = [int(s.shape[0]) for s in src_data]
        t["src_lengths"] = torch.tensor(src_lengths, dtype=torch.int64)
        t["src_size"] = int(sum(src_lengths))
        if packed and src_type == "text":
            t["packed_source"] = pack_sequences(src_data, src_pad, capacity_src, round_to)
    if tgt_data is not None:
        tgt_lengths = [int(s.shape[0]) for s in tgt_data]
        if padded:
            tgt_bt, _ = _pad_stack(tgt_data, tgt_pad)
            full = tgt_bt.t().contiguous()
            t["tgt_selfattn_mask"] = tgt_bt.eq(tgt_pad)
            t["target"] = full
            t["target_input"] = full[:-1]
            t["target_output"] = full[1:]
            t["target_input_selfattn_mask"] = full[:-1].t().eq(tgt_pad)
            t["target_pos"] = torch.arange(full.shape[0] - 1)[:, None].expand(-1, len(tgt_data)).contiguous()
            if create_reverse:
                rev = [torch.cat([s[:1], s[1:-1].flip(0), s[-1:]]) for s in tgt_data]
                rev_bt, _ = _pad_stack(rev, tgt_pad)
                t["target_rev"] = rev_bt
                t["target_input_rev"] = rev_bt.t()[:-1].contiguous()
                t["target_output_rev"] = rev_bt.t()[1:].contiguous()
        else:
            t["target"] = True
        t["tgt_lengths"] = torch.tensor(tgt_lengths, dtype=torch.int64)
        t["tgt_size"] = int(sum(n - 1 for n in tgt_lengths))
        if packed:
            pin = pack_sequences([s[:-1] for s in tgt_data], tgt_pad, capacity_tgt, round_to)
            pout = pack_sequences([s[1:] for s in tgt_data], tgt_pad, pin.tokens.numel(), 1)
            t["packed_target_input"] = pin
            t["packed_target_output"] = pout.tokens
    else:
        t["tgt_lengths"] = None
        t["tgt_size"] = 0
    t["size"] = len(src_data) if src_data is not None else len(tgt_data)
    if max_batch is not None and packed:
        # static batch dimension for graph capture: extend cu with empty sequences
        for k in ("packed_source", "packed_target_input"):
            if k in t:
                ps = t[k]
                extra = max_batch - ps.batch_size
                assert extra >= 0, "batch of %d sentences exceeds the static capacity %d" % (ps.batch_size, max_batch)
                if extra:
                    ps.cu = torch.cat([ps.cu, ps.cu[-1:].expand(extra)])
    if static_shapes and packed:
        for k in ("packed_source", "packed_target_input"):
            if k in t:
                t[k].max_len = bucket_max_len(t[k].max_len)
    for name, data in (("source_lang", src_lang), ("target_lang", tgt_lang), ("source_atbs", src_atb), ("target_atbs", tgt_atb)):
        if data is not None:
            t[name] = torch.cat([d.view(-1) for d in data]).long()
    t["indices"] = torch.tensor(index_data, dtype=torch.int64) if index_data is not None else None
    return Batch(t)


# ---------------------------------------------------------------------------------------------------
# Dataset
# ---------------------------------------------------------------------------------------------------
class Dataset(torch.utils.data.Dataset):
    """In-memory (or lazily indexed) parallel corpus with token-budget batches.

    ``src_data`` / ``tgt_data`` are sequences of tensors (anything indexable works: lists, mmap-backed
    datasets).  ``__getitem__`` returns a collated ``Batch`` so that a ``DataLoader`` can iterate over
    batch indices directly.
    """

    def __init__(self, src_data, tgt_data, src_sizes=None, tgt_sizes=None, src_langs=None, tgt_langs=None, src_atbs=None,
                 tgt_atbs=None, batch_size_words=2048, batch_size_frames=10 ** 12, batch_size_sents=10 ** 9, multiplier=1,
                 data_type="text", max_src_len=256, max_tgt_len=256, min_src_len=0, min_tgt_len=0, cleaning=True,
                 sorting=True, src_pad=C.PAD, tgt_pad=C.PAD, padded=True, packed=True, round_to=128, cut_off_size=256000,
                 smallest_batch_size=4, verbose=False, augmenter=None, create_reverse=False, past_src_data=None,
                 aux_tgt_data=None, static_shapes=False, concat=False, concat_seed=1234, **_ignored):
        self.src, self.tgt = src_data, tgt_data
        # ``concat``: every training example is extended with randomly drawn other examples, sources joined along time
        # and targets joined into one sentence, up to ``max_src_len`` (reference: onmt/data/dataset.py:863-865, 923-930,
        # 1285-1340 ``collater_concat``, :25-130 ``merge_concat_data``)
        self.concat = bool(concat)
        self.concat_max_len = int(max_src_len)
        concat_seed = int(concat_seed) % (2 ** 32)
        self.concat_rng = np.random.RandomState(concat_seed)
        self.aux_tgt = aux_tgt_data            # second target per example ("triangle" corpora)
        self.past_src = past_src_data          # previous source sentence per example (document-context models)
        self.src_langs, self.tgt_langs, self.src_atbs, self.tgt_atbs = src_langs, tgt_langs, src_atbs, tgt_atbs
        self.type = data_type
        self.src_pad, self.tgt_pad = src_pad, tgt_pad
        self.padded, self.packed, self.round_to = padded, packed, round_to
        self.create_reverse = create_reverse
        self.static_shapes = static_shapes     # round batch shapes so that training steps replay a few captured graphs
        self.augmenter = augmenter
        n = len(src_data) if src_data is not None else len(tgt_data)
        self.full_size = n
        size_of = lambda d: np.asarray([int(x.shape[0]) for x in d], dtype=np.int64)
        self.src_sizes = np.asarray(src_sizes, dtype=np.int64) if src_sizes is not None else (size_of(src_data) if src_data is not None else None)
        self.tgt_sizes = np.asarray(tgt_sizes, dtype=np.int64) if tgt_sizes is not None else (size_of(tgt_data) if tgt_data is not None else None)
        if self.src_sizes is not None and self.tgt_sizes is not None:
            lengths = np.maximum(self.src_sizes, self.tgt_sizes) if data_type == "text" else self.tgt_sizes
        else:
            lengths = self.src_sizes if self.src_sizes is not None else self.tgt_sizes
        order = np.arange(n, dtype=np.int64)
        if self.concat:
            # examples grow to about max_src_len each: a fixed number of them per batch, in random order
            order = np.random.RandomState(concat_seed).permutation(n).astype(np.int64)
            sorting = False
            per_batch = max(1, int(batch_size_frames // max(1, max_src_len))) if batch_size_frames < 10 ** 12 else \
                max(1, int(batch_size_words // max(1, max_src_len)))
            batch_size_sents = min(batch_size_sents, per_batch)
            batch_size_words = batch_size_frames = 10 ** 12
        if sorting:
            keys = []
            if self.tgt_sizes is not None:
                keys.append(self.tgt_sizes)
            if self.src_sizes is not None:
                keys.append(self.src_sizes)
            order = np.lexsort(tuple(keys)) if keys else order
        unbalanced = data_type != "text"
        self.batches = allocate_batches(order, lengths, self.src_sizes, self.tgt_sizes, batch_size_words, batch_size_frames,
                                        batch_size_sents, multiplier, max_src_len, max_tgt_len, min_src_len, min_tgt_len,
                                        cleaning, unbalanced, cut_off_size, smallest_batch_size)
        self.num_batches = len(self.batches)
        self.kept_ids = np.asarray(sorted({int(i) for b in self.batches for i in b}), dtype=np.int64)   # survived the length filters
        # static shapes: ONE sentence capacity for the whole data set (empty trailing sequences cost the attention kernels a
        # few loads each), so that the shape classes of the training step are (source tokens, target tokens) buckets only
        self.static_max_batch = bucket_capacity(max([len(b) for b in self.batches] + [1]), per_octave=4, floor=8)
        self.cur_index = 0
        self.batch_order = list(range(self.num_batches))
        if verbose:
            kept = sum(len(b) for b in self.batches)
            print("* %d sentences in %d batches (%d dropped by the length filters)" % (kept, self.num_batches, n - kept))

    def __len__(self):
        return self.num_batches

    def size(self):
        return self.full_size

    def batch_sizes(self) -> List[int]:
        return [len(b) for b in self.batches]

    def _concat_groups(self, ids, retries: int = 20):
        """For every example of the batch, the list of examples joined behind it: up to ``retries`` random candidates,
        shortest first, each taken if the joined source still fits and no example of the batch uses it already."""
        used = set(int(i) for i in ids)
        pool = self.kept_ids
        groups = []
        for i in ids:
            group, length = [int(i)], int(self.src_sizes[i])
            cand = pool[self.concat_rng.randint(0, len(pool), size=retries)]
            for c in sorted((int(c) for c in cand), key=lambda c: int(self.src_sizes[c])):
                L = int(self.src_sizes[c])
                if c not in used and length + L <= self.concat_max_len:
                    group.append(c)
                    used.add(c)
                    length += L
            groups.append(group)
        return groups

    def _get_concat_batch(self, ids) -> Batch:
        groups = self._concat_groups(ids)
        src = [torch.cat([torch.as_tensor(self.src[j]) for j in g], 0) for g in groups]

        def join_targets(g):
            # one sentence: the first example keeps its BOS, the last its EOS, everything in between loses both
            parts = [torch.as_tensor(self.tgt[j]) for j in g]
            inner = [p[(0 if k == 0 else 1):(len(p) if k == len(parts) - 1 else len(p) - 1)] for k, p in enumerate(parts)]
            return torch.cat(inner, 0)

        tgt = [join_targets(g) for g in groups]
        if self.augmenter is not None and self.type != "text":
            src = [self.augmenter.augment(s) for s in src]
        lang = lambda d: None if d is None else [(d[g[0]] if len(d) > 1 else d[0]) for g in groups]
        return collate(src, tgt, lang(self.src_langs), lang(self.tgt_langs), lang(self.src_atbs), lang(self.tgt_atbs),
                       self.src_pad, self.tgt_pad, self.type, [g[0] for g in groups], self.padded, self.packed,
                       round_to=self.round_to, create_reverse=self.create_reverse)

    def get_batch(self, index: int) -> Batch:
        ids = self.batches[index]
        if self.concat and self.src is not None and self.tgt is not None:
            return self._get_concat_batch(ids)
        pick = lambda d: None if d is None else [d[i] for i in ids]
        lang = lambda d: None if d is None else [(d[i] if len(d) > 1 else d[0]) for i in ids]
        src = pick(self.src)
        if self.augmenter is not None and src is not None and self.type != "text":
            src = [self.augmenter.augment(s) for s in src]
        return collate(src, pick(self.tgt), lang(self.src_langs), lang(self.tgt_langs), lang(self.src_atbs), lang(self.tgt_atbs),
                       self.src_pad, self.tgt_pad, self.type, ids, self.padded, self.packed, round_to=self.round_to,
                       create_reverse=self.create_reverse, past_src_data=pick(self.past_src), aux_tgt_data=pick(self.aux_tgt),
                       static_shapes=self.static_shapes,
                       max_batch=self.static_max_batch if (self.static_shapes and self.packed and self.type == "text") else None)

    __getitem__ = get_batch

    def get_collater(self):
        return lambda samples: samples[0] if len(samples) == 1 else samples

    def get_batches(self):
        return self.batches

    # sequential iteration (reference API: ``next`` / ``shuffle`` / ``reset``) ----------------------
    def shuffle(self, seed: Optional[int] = None):
        rng = np.random.RandomState(seed)
        self.batch_order = rng.permutation(self.num_batches).tolist()

    def reset(self):
        self.cur_index = 0

    def next(self, curriculum: bool = False):
        if self.cur_index >= self.num_batches:
            self.cur_index = 0
        b = self.get_batch(self.cur_index if curriculum else self.batch_order[self.cur_index])
        self.cur_index += 1
        return [b]
