#!/usr/bin/env python
"""python eval_autoencoder.py -model model.pt -autoencoder ae_e5.pt -src test.src [-tgt test.tgt] -output scores.txt
       [-batch_size 30] [-gpu -1]
Per-sentence reconstruction error of the auto-encoder trained by autoencoder.py on the hidden states of ``-model``
(the mean squared error over the sentence's state vectors), one number per input line.  (reference: eval_autoencoder.py)"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None):
    from autoencoder import hidden_states
    from nmtgminor_b200.data.dataset import collate
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import backward_compatible
    from nmtgminor_b200.tools.text import Autoencoder
    from nmtgminor_b200.train.checkpoint import load_model_state
    ap = argparse.ArgumentParser()
    ap.add_argument("-model", required=True)
    ap.add_argument("-autoencoder", required=True)
    ap.add_argument("-src", required=True)
    ap.add_argument("-tgt", default="")
    ap.add_argument("-output", default="pred.txt")
    ap.add_argument("-batch_size", type=int, default=30)
    ap.add_argument("-max_sent_length", type=int, default=2048)
    ap.add_argument("-gpu", type=int, default=-1)
    opt = ap.parse_args(argv)
    ckpt = torch.load(opt.model, map_location="cpu", weights_only=False)
    dicts = ckpt["dicts"]
    model = build_model(backward_compatible(ckpt["opt"]), dicts, remove_pretrain=True)
    load_model_state(model, ckpt["model"])
    blob = torch.load(opt.autoencoder, map_location="cpu", weights_only=False)
    ae = Autoencoder(blob["input_size"], blob["hidden_size"])
    ae.load_state_dict(blob["autoencoder"])
    representation = blob.get("representation", "EncoderHiddenState")
    dev = torch.device("cuda:%d" % opt.gpu) if opt.gpu >= 0 else torch.device("cpu")
    model, ae = model.to(dev).eval(), ae.to(dev).eval()
    src_lines = [l.split()[:opt.max_sent_length] for l in open(opt.src)]
    tgt_lines = [l.split()[:opt.max_sent_length] for l in open(opt.tgt)] if opt.tgt else [["<unk>"] for _ in src_lines]
    sd, td = dicts["src"], dicts["tgt"]
    with open(opt.output, "w") as out, torch.no_grad():
        for lo in range(0, len(src_lines), opt.batch_size):
            srcs = [sd.convert_to_idx(w, "<unk>") for w in src_lines[lo:lo + opt.batch_size]]
            tgts = [td.convert_to_idx(w, "<unk>", "<s>", "</s>") for w in tgt_lines[lo:lo + opt.batch_size]]
            batch = collate(srcs, tgts, round_to=1)
            if dev.type == "cuda":
                batch = batch.cuda(dev)
            x = hidden_states(model, batch, representation)
            err = ((ae(x) - x) ** 2).mean(-1)
            seqs = batch.packed_source() if representation.startswith("Encoder") else batch.packed_target_input()
            for i in range(len(srcs)):
                a, b = int(seqs.cu[i]), int(seqs.cu[i + 1])
                out.write("%.6f\n" % (float(err[a:b].mean()) if b > a else 0.0))
    print("wrote %d scores to %s" % (len(src_lines), opt.output))


if __name__ == "__main__":
    main()
