#!/usr/bin/env python
"""python extract_wav2vec2_codebook.py -model <ckpt> -src <wav list> -output out.codes [-kmeans km.pt] [-layer N]
Discrete units per frame: quantiser code indices or k-means clusters (reference: extract_wav2vec2_codebook.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.extract import main

if __name__ == "__main__":
    main(mode="codebook")
