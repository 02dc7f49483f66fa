#!/usr/bin/env python
"""python average_checkpoints_auto.py -models <directory or checkpoint prefix> [-top 10] [-output model.averaged]
       [-method mean|gmean] [-sort_by_date]
Average the best (by the perplexity in the file names) or the newest ``-top`` checkpoints of a run.
(reference: average_checkpoints_auto.py)"""
import argparse
import glob
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.checkpoints import average_checkpoints, best_checkpoints


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-models", required=True, help="directory with the checkpoints, or their common prefix")
    ap.add_argument("-type", default="seq2seq")
    ap.add_argument("-lm", action="store_true")
    ap.add_argument("-sort_by_date", action="store_true")
    ap.add_argument("-output", default="model.averaged")
    ap.add_argument("-gpu", type=int, default=-1)
    ap.add_argument("-top", type=int, default=10)
    ap.add_argument("-method", default="mean", choices=["mean", "gmean"])
    opt = ap.parse_args(argv)
    if opt.sort_by_date:
        pattern = os.path.join(opt.models, "*.pt") if os.path.isdir(opt.models) else opt.models + "*.pt"
        paths = sorted(glob.glob(pattern), key=os.path.getmtime, reverse=True)[:opt.top]
    else:
        prefix = os.path.join(opt.models, "") if os.path.isdir(opt.models) else opt.models
        paths = best_checkpoints(prefix, opt.top)
        if not paths and os.path.isdir(opt.models):
            # a directory: checkpoints of any prefix inside it
            names = sorted({f.split("_ppl_")[0] for f in os.listdir(opt.models) if "_ppl_" in f})
            for nme in names:
                paths += best_checkpoints(os.path.join(opt.models, nme), opt.top)
            paths = paths[:opt.top]
    if not paths:
        sys.exit("no checkpoints found under %s" % opt.models)
    print("\n".join(paths))
    average_checkpoints(paths, opt.output, opt.method)
    print("Saving averaged model to %s" % opt.output)


if __name__ == "__main__":
    main()
