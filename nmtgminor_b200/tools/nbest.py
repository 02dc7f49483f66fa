"""Pick the best hypothesis of every n-best block by a weighted sum of its scores.

    python -m nmtgminor_b200.tools.nbest -input nbest.txt -n_best 8 -coeff 1.0 0.3 -output pred.txt

Every input line is ``hypothesis ||| score_1 score_2 ...``; blocks of ``n_best`` consecutive lines belong to one source
sentence (the format ``translate.py -n_best`` and ``rescore.py`` write).  (reference: tools/get_best.py:36-76)"""
from __future__ import annotations

import argparse
from typing import Iterable, Iterator, Sequence


def pick_best(lines: Iterable[str], n_best: int, coeff: Sequence[float]) -> Iterator[str]:
    block = []
    for line in lines:
        line = line.rstrip("\n")
        if not line.strip():
            continue
        text, _, scores = line.partition(" ||| ")
        values = [float(s) for s in scores.split()]
        if len(values) > len(coeff):
            raise ValueError("%d scores on a line but %d coefficients" % (len(values), len(coeff)))
        block.append((sum(c * v for c, v in zip(coeff, values)), text.strip()))
        if len(block) == n_best:
            yield max(block, key=lambda t: t[0])[1]
            block = []
    if block:
        yield max(block, key=lambda t: t[0])[1]


def main(argv=None):
    ap = argparse.ArgumentParser(description="best hypothesis per n-best block")
    ap.add_argument("-input", required=True)
    ap.add_argument("-n_best", type=int, default=1)
    ap.add_argument("-output", default="pred.txt")
    ap.add_argument("-coeff", default=[1.0], nargs="+", type=float, help="one weight per score column")
    a = ap.parse_args(argv)
    with open(a.input) as fh, open(a.output, "w") as out:
        for best in pick_best(fh, a.n_best, a.coeff):
            out.write(best + "\n")


if __name__ == "__main__":
    main()
