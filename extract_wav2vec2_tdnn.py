#!/usr/bin/env python
"""python extract_wav2vec2_tdnn.py -model <ckpt> -src <wav list> -ark_output out.ark -scp_output out.scp [-layer N]
Frame-level features of a wav2vec 2.0 encoder in Kaldi ark / scp form (reference: extract_wav2vec2_tdnn.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.extract import main

if __name__ == "__main__":
    main(mode="tdnn")
