#!/usr/bin/env python
"""python quantize_kmeans.py --kmeans_model km.pt --features feats.pt --out_path units.txt [--deduplicate]
   python quantize_kmeans.py --kmeans_model km.pt --model speech_model.pt --wav_list wavs.txt --out_path units.txt [--layer 12]
Frame features (a list of [T, D] tensors, or frames taken from a speech encoder checkpoint on the fly) -> k-means unit ids,
one utterance per line.  (reference: quantize_kmeans.py, quantize_pretrained_hubert_kmeans.py)"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.kmeans import KMeans, quantize


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kmeans_model", "--kmeans_model_path", dest="kmeans_model", required=True)
    ap.add_argument("--features", default="", help="torch file with a list of [T, D] feature tensors")
    ap.add_argument("--model", "--acoustic_model_path", dest="model", default="", help="speech model checkpoint to take frames from")
    ap.add_argument("--wav_list", "--manifest_path", dest="wav_list", default="", help="one '<id> <wav path>' per line")
    ap.add_argument("--layer", type=int, default=-1)
    ap.add_argument("--out_path", "--out_quantized_file_path", dest="out_path", required=True)
    ap.add_argument("--deduplicate", action="store_true", help="merge runs of the same unit")
    ap.add_argument("--gpu", type=int, default=-1)
    opt = ap.parse_args(argv)
    km = KMeans.load(torch.load(opt.kmeans_model, weights_only=False))
    dev = "cuda:%d" % opt.gpu if opt.gpu >= 0 else "cpu"
    with open(opt.out_path, "w") as out:
        if opt.features:
            for f in torch.load(opt.features, weights_only=False):
                out.write(" ".join(map(str, quantize(km, f, opt.deduplicate))) + "\n")
        else:
            from nmtgminor_b200.tools.extract import encoder_frames, load_speech_encoder, read_wav_list
            enc, _ = load_speech_encoder(opt.model, dev)
            for uid, wav in read_wav_list(opt.wav_list):
                frames = encoder_frames(enc, [wav], opt.layer if opt.layer >= 0 else None, dev)[0]
                out.write("%s|%s\n" % (uid, " ".join(map(str, quantize(km, frames.float().cpu(), opt.deduplicate)))))


if __name__ == "__main__":
    main()
