#!/usr/bin/env python
"""Preprocessing for "triangle" corpora: every example has a source, a target and an auxiliary target (for instance
audio, translation and transcript).

    python preprocess_triangle.py -train_src s -train_tgt t -aux_train_tgt a -valid_src vs -valid_tgt vt -aux_valid_tgt va \\
           -save_data out [-format raw|mmap] [-asr ...]

The auxiliary side gets its own vocabulary (``dicts['aux_tgt']``) and is stored as ``aux_tgt`` next to ``tgt`` with the
same line filter, so the three sides stay aligned (reference: preprocess_triangle.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import preprocess


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if "-aux_train_tgt" not in argv:
        raise SystemExit("preprocess_triangle.py needs -aux_train_tgt (and -aux_valid_tgt)")
    return preprocess.main(argv)


if __name__ == "__main__":
    main()
