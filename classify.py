#!/usr/bin/env python
"""Label every line (or utterance) of a file with a trained classifier.

    python classify.py -model classifier.pt -src input.txt [-output pred.txt] [-gpu 0] [-batch_size 32]

Writes one predicted label per input line; with ``-tgt labels.txt`` also prints the accuracy (reference: classify.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.inference.scoring import ClassifierPredictor
from nmtgminor_b200.options import make_translate_parser


def main(argv=None):
    opt = make_translate_parser().parse_args(argv)
    predictor = ClassifierPredictor(opt)
    src = [l.split() for l in open(opt.src, encoding="utf-8")]
    out = open(opt.output, "w", encoding="utf-8") if getattr(opt, "output", None) and opt.output != "stdout" else sys.stdout
    preds = predictor.predict(src, batch_size=max(1, getattr(opt, "batch_size", 32)))
    names = [predictor.label_name(i) for i, _ in preds]
    for name, (_, logp) in zip(names, preds):
        out.write("%s\t%.4f\n" % (name, logp) if getattr(opt, "verbose", False) else name + "\n")
    if getattr(opt, "tgt", None):
        gold = [l.strip() for l in open(opt.tgt, encoding="utf-8")]
        hits = sum(1 for g, n in zip(gold, names) if g == n)
        print("accuracy: %.4f (%d / %d)" % (hits / max(len(gold), 1), hits, len(gold)), file=sys.stderr)
    if out is not sys.stdout:
        out.close()


if __name__ == "__main__":
    main()
