#!/usr/bin/env python
"""python sample_lm.py -models lm.pt [-prefix "the cat"] [-n 5] [-max_len 50] [-temperature 1.0] [-top_k 0] [-seed 0] [-gpu -1]
Draw continuations from a language model trained with train_language_model.py.  With several checkpoints separated by |
and -output, the models are averaged instead, which is what the reference's script of this name does
(reference: sample_lm.py:24-126)."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-models", required=True)
    ap.add_argument("-output", default="")
    ap.add_argument("-method", default="mean", choices=["mean", "gmean"])
    ap.add_argument("-gpu", type=int, default=-1)
    ap.add_argument("-prefix", default="")
    ap.add_argument("-n", type=int, default=1)
    ap.add_argument("-max_len", type=int, default=50)
    ap.add_argument("-temperature", type=float, default=1.0)
    ap.add_argument("-top_k", type=int, default=0)
    ap.add_argument("-seed", type=int, default=0)
    opt = ap.parse_args(argv)
    paths = opt.models.split("|")
    if len(paths) > 1 or opt.output:
        from nmtgminor_b200.tools.checkpoints import average_checkpoints
        out = opt.output or "model.averaged"
        average_checkpoints(paths, out, opt.method)
        print("Saving averaged model to %s" % out)
        return
    from nmtgminor_b200.models.factory import build_language_model
    from nmtgminor_b200.options import backward_compatible
    from nmtgminor_b200.tools.text import sample_lm
    from nmtgminor_b200.train.checkpoint import load_model_state
    ckpt = torch.load(paths[0], map_location="cpu", weights_only=False)
    model_opt = backward_compatible(ckpt["opt"])
    model = build_language_model(model_opt, ckpt["dicts"])
    load_model_state(model, ckpt["model"])
    if opt.gpu >= 0:
        model = model.cuda(opt.gpu)
    model.eval()
    d = ckpt["dicts"]["tgt"]
    for i in range(opt.n):
        words = sample_lm(model, d, opt.prefix.split(), opt.max_len, opt.temperature, opt.top_k, opt.seed + i)
        print(" ".join(words))


if __name__ == "__main__":
    main()
