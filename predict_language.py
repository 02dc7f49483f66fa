#!/usr/bin/env python
"""Predict the language of every input line with a model that carries a language-identification head.

    python predict_language.py -model m.pt -src input.txt [-output langs.txt] [-gpu 0] [-batch_size 32]

Writes one language id per line (reference: predict_language.py, onmt/inference/predictor.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.inference.scoring import LanguagePredictor
from nmtgminor_b200.options import make_translate_parser


def main(argv=None):
    opt = make_translate_parser().parse_args(argv)
    predictor = LanguagePredictor(opt)
    src = [l.split() for l in open(opt.src, encoding="utf-8")]
    out = open(opt.output, "w", encoding="utf-8") if getattr(opt, "output", None) and opt.output != "stdout" else sys.stdout
    bs = max(1, getattr(opt, "batch_size", 32))
    for i in range(0, len(src), bs):
        for lang in predictor.predict(src[i:i + bs]):
            out.write("%s\n" % lang)
    if out is not sys.stdout:
        out.close()


if __name__ == "__main__":
    main()
