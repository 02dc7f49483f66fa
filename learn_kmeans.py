#!/usr/bin/env python
"""python learn_kmeans.py <features.pt (list of [T, D] tensors)> <n_clusters> <out.pt>     (reference: learn_kmeans.py)
python learn_kmeans.py quantize <kmeans.pt> <features.pt> <out.txt>                      (reference: quantize_kmeans.py)"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.kmeans import KMeans, learn_kmeans, quantize

if __name__ == "__main__":
    if sys.argv[1] == "quantize":
        km = KMeans.load(torch.load(sys.argv[2]))
        with open(sys.argv[4], "w") as fh:
            for f in torch.load(sys.argv[3]):
                fh.write(" ".join(map(str, quantize(km, f))) + "\n")
    else:
        feats = torch.load(sys.argv[1])
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        torch.save(learn_kmeans(feats, int(sys.argv[2]), device=dev).state_dict(), sys.argv[3])
