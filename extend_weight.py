#!/usr/bin/env python
"""python extend_weight.py -model model.pt -n_languages 12 [-output out.pt]
More languages for a multilingual checkpoint: every per-language parameter (factorised / partitioned weight factors,
language embeddings, per-language LayerNorm, adapters) gets slices for the new languages; the rest of the model, the
dictionaries and the options are copied.  (reference: extend_weight.py)"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.languages import extend_languages


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-model", required=True)
    ap.add_argument("-output", default="")
    ap.add_argument("-n_languages", type=int, default=10)
    ap.add_argument("-gpu", type=int, default=-1, help="accepted for compatibility; the work is done on the CPU")
    opt = ap.parse_args(argv)
    ckpt = torch.load(opt.model, map_location="cpu", weights_only=False)
    langs = ckpt["dicts"].get("langs") or {}
    n_old = max(len(langs), 1)
    touched = extend_languages(ckpt["model"], n_old, opt.n_languages)
    ckpt.update(optim=None, epoch=-1, iteration=-1, batchOrder=None)
    out = opt.output or "%s.extend%d" % (opt.model, opt.n_languages)
    torch.save(ckpt, out)
    print("extended %d tensors from %d to %d languages -> %s" % (len(touched), n_old, opt.n_languages, out))


if __name__ == "__main__":
    main()
