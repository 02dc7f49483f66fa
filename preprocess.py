#!/usr/bin/env python
"""Corpus preprocessing: vocabularies + binarised train/valid sets.

Writes, for ``-save_data <name>``:
  * ``-format raw`` / ``bin``:  ``<name>.train.pt`` = {'dicts', 'type', 'train': {'src','tgt','src_sizes','tgt_sizes',
    'src_lang','tgt_lang'}, 'valid': {...}} (lists of id tensors);
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
from nmtgminor_b200.data.binarizer import Tokenizer, binarize_file
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


def make_data(src_file, tgt_file, src_dict, tgt_dict, opt, tokenizer):
    src = binarize_file(src_file, src_dict, tokenizer, None, None, opt.num_threads) if src_file else None
    tgt = binarize_file(tgt_file, tgt_dict, tokenizer, C.BOS_WORD, C.EOS_WORD, opt.num_threads) if tgt_file else None
    n = len(src["data"]) if src else len(tgt["data"])
    keep = []
    for i in range(n):
        ls = src["sizes"][i] if src else 1
        lt = tgt["sizes"][i] - 2 if tgt else 1
        if 0 < ls <= opt.src_seq_length and 0 < lt <= opt.tgt_seq_length:
            keep.append(i)
    pick = lambda d: None if d is None else {"data": [d["data"][i] for i in keep], "sizes": [d["sizes"][i] for i in keep]}
    print("Prepared %d sentences (%d ignored due to length)" % (len(keep), n - len(keep)))
    return pick(src), pick(tgt)


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
    langs = {}
    for l in (getattr(opt, "train_src_lang", "src") or "src").split("|") + (getattr(opt, "train_tgt_lang", "tgt") or "tgt").split("|"):
        langs.setdefault(l, len(langs))
    dicts["langs"] = langs
    dicts["atbs"] = {"nothingness": 0}

    sets = {}
    for split, sfiles, tfiles in (("train", train_src, train_tgt),
                                  ("valid", opt.valid_src.split("|") if opt.valid_src else [],
                                   opt.valid_tgt.split("|") if opt.valid_tgt else [])):
        src_all, tgt_all = {"data": [], "sizes": []}, {"data": [], "sizes": []}
        for i in range(max(len(sfiles), len(tfiles))):
            s, t = make_data(sfiles[i] if i < len(sfiles) else None, tfiles[i] if i < len(tfiles) else None,
                             dicts.get("src"), dicts["tgt"], opt, tokenizer)
            for acc, part in ((src_all, s), (tgt_all, t)):
                if part is not None:
                    acc["data"] += part["data"]
                    acc["sizes"] += part["sizes"]
        sets[split] = {"src": src_all["data"] or None, "tgt": tgt_all["data"] or None,
                       "src_sizes": src_all["sizes"] or None, "tgt_sizes": tgt_all["sizes"] or None,
                       "src_lang": [torch.tensor([0])], "tgt_lang": [torch.tensor([1 if len(langs) > 1 else 0])]}

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
        print("Saved mmap data to %s.*" % opt.save_data)
    else:
        raise NotImplementedError("format %r: audio formats are handled by preprocess with -asr (scp / wav lists)" % fmt)


if __name__ == "__main__":
    main()
