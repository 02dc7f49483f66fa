#!/usr/bin/env python
"""Score or re-rank hypotheses with a trained model.

    python rescore.py -model m.pt -src src.txt -tgt hyp.txt [-gpu 0] [-alpha 0.6] [-n_best N] [-output out.txt]

With ``-n_best N`` the target file holds N consecutive hypotheses per source line and the best one per line is
written; otherwise one score per line and the corpus perplexity are printed (reference: rescore.py,
tools/perplexity_score.py, onmt/Rescorer.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.inference.scoring import PerplexityScorer, Rescorer
from nmtgminor_b200.options import make_translate_parser


def main(argv=None):
    opt = make_translate_parser().parse_args(argv)
    src = [l.split() for l in open(opt.src, encoding="utf-8")]
    tgt = [l.split() for l in open(opt.tgt, encoding="utf-8")]
    out = open(opt.output, "w", encoding="utf-8") if getattr(opt, "output", None) and opt.output != "stdout" else sys.stdout
    n = max(1, getattr(opt, "n_best", 1))
    if n > 1:
        nbest = [tgt[i * n:(i + 1) * n] for i in range(len(src))]
        for ranked in Rescorer(opt).rescore(src, nbest, alpha=getattr(opt, "alpha", 0.0)):
            out.write(" ".join(ranked[0][0]) + "\n")
    else:
        scores, ppl = PerplexityScorer(opt).score(src, tgt, batch_size=getattr(opt, "batch_size", 32))
        for s in scores:
            out.write("%.4f\n" % s)
        print("perplexity: %.4f" % ppl, file=sys.stderr)


if __name__ == "__main__":
    main()
