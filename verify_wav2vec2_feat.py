#!/usr/bin/env python
"""python verify_wav2vec2_feat.py -model <ckpt> -src <wav list> -scp stored.scp [-layer N] [-gpu 0]
Recomputes wav2vec 2.0 features and checks them against a Kaldi scp / ark dump written by extract_wav2vec2_tdnn.py
(reference: verify_wav2vec2_feat.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.extract import main

if __name__ == "__main__":
    main(mode="verify")
