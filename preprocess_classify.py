#!/usr/bin/env python
"""Preprocessing for classification corpora: the target side is a label (or a label sequence) per example, stored without
sentence delimiters; the target "vocabulary" is the label set.

    python preprocess_classify.py -train_src s -train_tgt labels -valid_src vs -valid_tgt vlabels -save_data out [-asr ...]

Same options as ``preprocess.py`` with ``-classification`` switched on (reference: preprocess_classify.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import preprocess


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if "-classification" not in argv:
        argv.append("-classification")
    return preprocess.main(argv)


if __name__ == "__main__":
    main()
