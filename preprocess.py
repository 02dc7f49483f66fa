#!/usr/bin/env python
"""Corpus preprocessing: vocabularies + binarised train/valid sets.

Writes, for ``-save_data <name>``:
  * ``-format raw`` / ``bin``:  ``<name>.train.pt`` = {'dicts', 'type', 'train': {'src','tgt','src_sizes','tgt_sizes',
    'src_lang','tgt_lang'}, 'valid': {...}} (lists of id tensors);
  * ``-asr -asr_format wav|scp -format wav|scp|scpmem``: ``<name>.dict.pt``, ``<name>.{wav,scp}_path.pt`` (utterance index
    ``{'train': [...], 'valid': [...]}`` of ``(path, start, end, sample_rate)`` / ``(ark, offset)`` entries), memory-mapped
    targets and ``*_sizes.npy``;
  * ``-format mmap`` / ``mmem``: ``<name>.dict.pt`` plus ``<name>.{train,valid}.{src,tgt,src_lang,tgt_lang}.{bin,idx}`` in
    the MMIDIDX layout and ``<name>.{train,valid}.{src,tgt}_sizes.npy``.
Same option names and file layouts as the reference (preprocess.py:27-170 options, :1261-1265 save).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import numpy as np
import torch

from nmtgminor_b200 import constants as C
from nmtgminor_b200.data.binarizer import Tokenizer, binarize_file, binarize_speech_file
from nmtgminor_b200.data.mmap_dataset import best_dtype, write_dataset
from nmtgminor_b200.dictionary import Dict
from nmtgminor_b200.options import make_preprocess_parser


def make_vocab(name, files, size, tokenizer, lower=False, specials=(C.PAD_WORD, C.UNK_WORD, C.BOS_WORD, C.EOS_WORD)):
    counters = [Dict.count_file(f, tokenizer, lower) for f in files]
    vocab = Dict.build(counters, size, specials, lower)
    print("Created %s dictionary of size %d" % (name, vocab.size()))
    return vocab


def init_vocab(name, files, vocab_file, size, tokenizer, lower=False):
    if vocab_file:
        print("Reading %s vocabulary from %s" % (name, vocab_file))
        vocab = Dict(lower=lower)
        vocab.add_specials([C.PAD_WORD, C.UNK_WORD, C.BOS_WORD, C.EOS_WORD])
        with open(vocab_file, encoding="utf-8") as fh:
            for line in fh:
                if line.strip():
                    vocab.add(line.split()[0])
        return vocab
    return make_vocab(name, files, size, tokenizer, lower)


def make_data(src_file, tgt_file, src_dict, tgt_dict, opt, tokenizer, aux_file=None, aux_dict=None):
    """Binarises one (source, target[, auxiliary target]) file group and drops the lines whose lengths are out of range.
    ``-classification``: the target is a label sequence without sentence delimiters (reference: preprocess_classify.py:184).
    ``aux_file``: a second target side kept aligned with the first (reference: preprocess_triangle.py, ``-aux_train_tgt``)."""
    external = None
    if getattr(opt, "external_tokenizer", ""):
        from nmtgminor_b200.data.binarizer import load_external_tokenizer
        external = load_external_tokenizer(opt.external_tokenizer)
    if getattr(opt, "asr", False):
        # audio source: an index of utterances (wav segments or Kaldi matrices), never the samples themselves
        src = binarize_speech_file(src_file, getattr(opt, "asr_format", "wav") or "wav", getattr(opt, "num_mel_bin", 0) or 0,
                                   getattr(opt, "concat", 1) or 1) if src_file else None
    else:
        src = binarize_file(src_file, src_dict, tokenizer, None, None, opt.num_threads, external=external) if src_file else None
    # an external tokenizer adds its own sentence delimiters
    labels = getattr(opt, "classification", False)
    delim = (None, None) if (external or labels) else (C.BOS_WORD, C.EOS_WORD)
    tgt = binarize_file(tgt_file, tgt_dict, tokenizer, delim[0], delim[1], opt.num_threads, external=external) if tgt_file else None
    aux = binarize_file(aux_file, aux_dict, tokenizer, C.BOS_WORD, C.EOS_WORD, opt.num_threads) if aux_file else None
    n = len(src["data"]) if src else len(tgt["data"])
    if aux is not None:
        assert len(aux["data"]) == n, "the auxiliary target file has %d lines, the corpus %d" % (len(aux["data"]), n)
    keep = []
    for i in range(n):
        ls = src["sizes"][i] if src else 1
        lt = (tgt["sizes"][i] - (0 if labels else 2)) if tgt else 1
        src_ok = ls > 0 if getattr(opt, "asr", False) else 0 < ls <= opt.src_seq_length   # audio is not length-filtered here
        if src_ok and 0 < lt <= opt.tgt_seq_length:
            keep.append(i)
    pick = lambda d: None if d is None else {"data": [d["data"][i] for i in keep], "sizes": [d["sizes"][i] for i in keep]}
    print("Prepared %d sentences (%d ignored due to length)" % (len(keep), n - len(keep)))
    if aux_file:
        return pick(src), pick(tgt), pick(aux)
    return pick(src), pick(tgt)


def write_multi_dataset(opt, dicts, langs, tokenizer):
    """``-multi_dataset``: every (source file, target file) pair becomes its own data set in a sibling directory
    ``train.<i>.<src lang>-<tgt lang>/data.*`` (``valid.<i>.…`` likewise) next to ``<save_data>.dict.pt``; the trainer
    iterates them jointly (reference layout: train_distributed.py:487-545)."""
    root = os.path.dirname(os.path.abspath(opt.save_data))
    os.makedirs(root, exist_ok=True)
    torch.save(dicts, opt.save_data + ".dict.pt")
    asr = getattr(opt, "asr", False)
    fmt = getattr(opt, "format", "mmap")
    for split, s_arg, t_arg, sl_arg, tl_arg in (("train", opt.train_src, opt.train_tgt, getattr(opt, "train_src_lang", "src"),
                                                 getattr(opt, "train_tgt_lang", "tgt")),
                                                ("valid", opt.valid_src, opt.valid_tgt, getattr(opt, "valid_src_lang", "src"),
                                                 getattr(opt, "valid_tgt_lang", "tgt"))):
        sfiles = s_arg.split("|") if s_arg else []
        tfiles = t_arg.split("|") if t_arg else []
        slangs = (sl_arg or "src").split("|")
        tlangs = (tl_arg or "tgt").split("|")
        for i in range(max(len(sfiles), len(tfiles))):
            sl = slangs[i] if i < len(slangs) else slangs[-1]
            tl = tlangs[i] if i < len(tlangs) else tlangs[-1]
            for l in (sl, tl):
                langs.setdefault(l, len(langs))
            s, t = make_data(sfiles[i] if i < len(sfiles) else None, tfiles[i] if i < len(tfiles) else None,
                             dicts.get("src"), dicts["tgt"], opt, tokenizer)
            d = os.path.join(root, "%s.%d.%s-%s" % (split, i, sl, tl))
            os.makedirs(d, exist_ok=True)
            if s is not None:
                if asr:
                    torch.save(s["data"], os.path.join(d, "data.scp_path.pt"))       # the reference uses this name for wav lists too
                else:
                    write_dataset(os.path.join(d, "data.src"), s["data"], best_dtype(dicts["src"].size()))
                np.save(os.path.join(d, "data.src_sizes.npy"), np.asarray(s["sizes"]))
            if t is not None:
                write_dataset(os.path.join(d, "data.tgt"), t["data"], best_dtype(dicts["tgt"].size()))
                np.save(os.path.join(d, "data.tgt_sizes.npy"), np.asarray(t["sizes"]))
            write_dataset(os.path.join(d, "data.src_lang"), [torch.tensor([langs[sl]])], np.int32)
            write_dataset(os.path.join(d, "data.tgt_lang"), [torch.tensor([langs[tl]])], np.int32)
            print("Saved %s set %d (%s-%s, %s) to %s" % (split, i, sl, tl, fmt, d))
    torch.save(dicts, opt.save_data + ".dict.pt")      # the language table may have grown


def main(argv=None):
    opt = make_preprocess_parser().parse_args(argv)
    torch.manual_seed(getattr(opt, "seed", 3435))
    tokenizer = Tokenizer(getattr(opt, "input_type", "word"), getattr(opt, "lower", False))
    train_src = opt.train_src.split("|") if opt.train_src else []
    train_tgt = opt.train_tgt.split("|") if opt.train_tgt else []
    dicts = {}
    if getattr(opt, "join_vocab", False):
        dicts["src"] = dicts["tgt"] = init_vocab("joined", train_src + train_tgt, opt.tgt_vocab or opt.src_vocab,
                                                 opt.tgt_vocab_size, tokenizer, opt.lower)
    else:
        if train_src and not getattr(opt, "asr", False):
            dicts["src"] = init_vocab("source", train_src, opt.src_vocab, opt.src_vocab_size, tokenizer, opt.lower)
        dicts["tgt"] = init_vocab("target", train_tgt, opt.tgt_vocab, opt.tgt_vocab_size, tokenizer, opt.lower)
    aux_train = opt.aux_train_tgt.split("|") if getattr(opt, "aux_train_tgt", "") else []
    aux_valid = opt.aux_valid_tgt.split("|") if getattr(opt, "aux_valid_tgt", "") else []
    if aux_train:
        dicts["aux_tgt"] = init_vocab("auxiliary target", aux_train, getattr(opt, "aux_tgt_vocab", ""), opt.tgt_vocab_size,
                                      tokenizer, opt.lower)
    langs = {}
    for l in (getattr(opt, "train_src_lang", "src") or "src").split("|") + (getattr(opt, "train_tgt_lang", "tgt") or "tgt").split("|"):
        langs.setdefault(l, len(langs))
    dicts["langs"] = langs
    dicts["atbs"] = {"nothingness": 0}

    if getattr(opt, "multi_dataset", False):
        return write_multi_dataset(opt, dicts, langs, tokenizer)

    sets = {}
    for split, sfiles, tfiles, afiles in (("train", train_src, train_tgt, aux_train),
                                          ("valid", opt.valid_src.split("|") if opt.valid_src else [],
                                           opt.valid_tgt.split("|") if opt.valid_tgt else [], aux_valid)):
        src_all, tgt_all, aux_all = {"data": [], "sizes": []}, {"data": [], "sizes": []}, {"data": [], "sizes": []}
        for i in range(max(len(sfiles), len(tfiles))):
            parts = make_data(sfiles[i] if i < len(sfiles) else None, tfiles[i] if i < len(tfiles) else None,
                              dicts.get("src"), dicts["tgt"], opt, tokenizer,
                              aux_file=afiles[i] if i < len(afiles) else None, aux_dict=dicts.get("aux_tgt"))
            for acc, part in zip((src_all, tgt_all, aux_all), parts):
                if part is not None:
                    acc["data"] += part["data"]
                    acc["sizes"] += part["sizes"]
        sets[split] = {"src": src_all["data"] or None, "tgt": tgt_all["data"] or None,
                       "src_sizes": src_all["sizes"] or None, "tgt_sizes": tgt_all["sizes"] or None,
                       "src_lang": [torch.tensor([0])], "tgt_lang": [torch.tensor([1 if len(langs) > 1 else 0])]}
        if aux_all["data"]:
            sets[split]["aux_tgt"], sets[split]["aux_tgt_sizes"] = aux_all["data"], aux_all["sizes"]

    fmt = getattr(opt, "format", "raw")
    os.makedirs(os.path.dirname(os.path.abspath(opt.save_data)), exist_ok=True)
    if fmt in ("raw", "bin"):
        out = {"dicts": dicts, "type": getattr(opt, "src_type", "text"), "train": sets["train"], "valid": sets["valid"]}
        torch.save(out, opt.save_data + ".train.pt")
        print("Saved data to %s.train.pt" % opt.save_data)
    elif fmt in ("mmap", "mmem"):
        torch.save(dicts, opt.save_data + ".dict.pt")
        for split in ("train", "valid"):
            for side in ("src", "tgt"):
                data = sets[split][side]
                if data is None:
                    continue
                vocab = dicts.get(side)
                write_dataset("%s.%s.%s" % (opt.save_data, split, side), data, best_dtype(vocab.size() if vocab else None))
                np.save("%s.%s.%s_sizes.npy" % (opt.save_data, split, side), np.asarray(sets[split][side + "_sizes"]))
            for side in ("src_lang", "tgt_lang"):
                write_dataset("%s.%s.%s" % (opt.save_data, split, side), sets[split][side], np.int32)
            if sets[split].get("aux_tgt"):
                write_dataset("%s.%s.aux_tgt" % (opt.save_data, split), sets[split]["aux_tgt"], best_dtype(dicts["aux_tgt"].size()))
                np.save("%s.%s.aux_tgt_sizes.npy" % (opt.save_data, split), np.asarray(sets[split]["aux_tgt_sizes"]))
        print("Saved mmap data to %s.*" % opt.save_data)
    elif fmt in ("wav", "scp", "scpmem"):
        # audio: <name>.{wav,scp}_path.pt = {'train': entries, 'valid': entries}; targets memory-mapped; sizes as .npy
        assert getattr(opt, "asr", False), "-format %s needs -asr (the source side is an utterance list)" % fmt
        torch.save(dicts, opt.save_data + ".dict.pt")
        torch.save({"train": sets["train"]["src"], "valid": sets["valid"]["src"]},
                   opt.save_data + (".wav_path.pt" if fmt == "wav" else ".scp_path.pt"))
        for split in ("train", "valid"):
            if sets[split]["tgt"] is not None:
                write_dataset("%s.%s.tgt" % (opt.save_data, split), sets[split]["tgt"], best_dtype(dicts["tgt"].size()))
            for side in ("src", "tgt"):
                if sets[split][side + "_sizes"] is not None:
                    np.save("%s.%s.%s_sizes.npy" % (opt.save_data, split, side), np.asarray(sets[split][side + "_sizes"]))
            for side in ("src_lang", "tgt_lang"):
                write_dataset("%s.%s.%s" % (opt.save_data, split, side), sets[split][side], np.int32)
        print("Saved %s utterance index and targets to %s.*" % (fmt, opt.save_data))
    else:
        raise NotImplementedError("format %r" % fmt)


if __name__ == "__main__":
    main()
