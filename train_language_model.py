#!/usr/bin/env python
"""Train a decoder-only language model:  python train_language_model.py -data corpus -model transformer_xl_lm ...
The data are the target side of a preprocessed corpus (``preprocess.py -lm``); the model family defaults to the
Transformer-XL language model (reference: train_language_model.py, onmt/models/transformer_xl.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from train_distributed import cli_main

if __name__ == "__main__":
    argv = sys.argv[1:]
    if "-model" not in argv:
        argv += ["-model", "transformer_xl_lm"]
    cli_main(argv)
