#!/usr/bin/env python
"""Train an utterance classifier (language / accent id):  python train_classify.py -data corpus -model classifier ...
(reference: train_classify.py, onmt/train_utils/classify_trainer.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from train_distributed import cli_main

if __name__ == "__main__":
    argv = sys.argv[1:]
    if "-model" not in argv:
        argv += ["-model", "classifier"]
    cli_main(argv)
