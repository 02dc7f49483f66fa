#!/usr/bin/env python
"""python rematch_language_embedding.py -model_src a.pt -model_tgt b.pt -model_out out.pt
The language tables of checkpoint a (language embeddings, partition factors) re-ordered to the language dictionary of
checkpoint b, which also becomes the dictionary of the output.  (reference: rematch_language_embedding.py)"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.languages import _TABLES, rematch_language_table


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-model_src", required=True)
    ap.add_argument("-model_tgt", required=True)
    ap.add_argument("-model_out", required=True)
    opt = ap.parse_args(argv)
    src = torch.load(opt.model_src, map_location="cpu", weights_only=False)
    tgt = torch.load(opt.model_tgt, map_location="cpu", weights_only=False)
    old, new = src["dicts"].get("langs") or {}, tgt["dicts"].get("langs") or {}
    n = 0
    for name, w in list(src["model"].items()):
        if _TABLES.search(name) and torch.is_tensor(w) and w.dim() >= 1 and w.shape[0] == max(len(old), 1):
            src["model"][name] = rematch_language_table(w, old, new)
            n += 1
    for lang in old:
        if lang in new:
            print(lang, old[lang], "->", new[lang])
    src["dicts"] = tgt["dicts"]
    src.update(optim=None, epoch=-1, iteration=-1, batchOrder=None)
    torch.save(src, opt.model_out)
    print("re-ordered %d language tables -> %s" % (n, opt.model_out))


if __name__ == "__main__":
    main()
