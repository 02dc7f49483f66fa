#!/usr/bin/env python
"""Single entry point for training; identical to ``train_distributed.py`` (which handles 1..N GPUs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from train_distributed import cli_main

if __name__ == "__main__":
    cli_main()
