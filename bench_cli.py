#!/usr/bin/env python
"""Throughput of the product command line (``preprocess.py`` -> ``train_distributed.py``) on a synthetic corpus of the
benchmark's shape, to be compared with ``bench.py``'s end-to-end number: what a user of the CLI gets, data loader,
shuffling, logging and all.

    python bench_cli.py [--gpus N] [--updates 1400] [--sentences 60000] [--tiny]

Writes a synthetic parallel corpus (sentence lengths uniform in [20, 100], vocabulary of 32 000 words, the corpus
``bench.py`` draws its batches from), binarises it with ``preprocess.py``, trains Transformer-big with the trainer's
defaults for CUDA (bf16, CUDA graphs per batch shape class, peer-memory data parallelism for N > 1) for ``--updates``
updates, and reports the median target tokens / s of the trainer's own log windows over the second half of the run (a
shape class is captured into a CUDA graph at its eighth batch, so the first epochs run partly kernel by kernel).  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def write_corpus(d: str, n: int, vocab: int, lo: int, hi: int, seed: int = 1):
    rng = np.random.RandomState(seed)
    for split, count in (("train", n), ("valid", max(64, n // 100))):
        for side in ("src", "tgt"):
            with open(os.path.join(d, "%s.%s" % (split, side)), "w") as fh:
                for _ in range(count):
                    L = int(rng.randint(lo, hi + 1))
                    fh.write(" ".join("w%d" % w for w in rng.randint(0, vocab, size=L)) + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--updates", type=int, default=1400)
    ap.add_argument("--sentences", type=int, default=60000)
    ap.add_argument("--tiny", action="store_true", help="small model and corpus (CPU dry run)")
    ap.add_argument("--keep", default="", help="directory to keep the corpus and the log in")
    args = ap.parse_args()
    import torch
    cuda = torch.cuda.is_available() and not args.tiny
    tmp = args.keep or tempfile.mkdtemp(prefix="nmtg_cli_")
    os.makedirs(tmp, exist_ok=True)
    vocab, lo, hi = (32000 - 4, 20, 100) if not args.tiny else (200, 5, 12)
    n = args.sentences if not args.tiny else 400
    write_corpus(tmp, n, vocab, lo, hi)
    prefix = os.path.join(tmp, "data")
    py = sys.executable
    subprocess.run([py, os.path.join(HERE, "preprocess.py"), "-train_src", os.path.join(tmp, "train.src"), "-train_tgt",
                    os.path.join(tmp, "train.tgt"), "-valid_src", os.path.join(tmp, "valid.src"), "-valid_tgt",
                    os.path.join(tmp, "valid.tgt"), "-save_data", prefix, "-format", "raw", "-join_vocab",
                    "-src_seq_length", "128", "-tgt_seq_length", "128"], check=True, stdout=subprocess.DEVNULL)
    size = ["-model_size", "1024", "-inner_size", "4096", "-n_heads", "16", "-layers", "6"] if not args.tiny else \
        ["-model_size", "64", "-inner_size", "128", "-n_heads", "2", "-layers", "1"]
    every = max(1, args.updates // 16)
    cmd = [py, os.path.join(HERE, "train_distributed.py"), "-data", prefix, "-data_format", "raw", "-save_model",
           os.path.join(tmp, "model"), "-model", "transformer", "-tie_weights", "-join_embedding", "-ffn_activation", "relu",
           "-batch_size_words", "13000" if not args.tiny else "300", "-batch_size_sents", "100000", "-batch_size_multiplier", "8",
           "-max_src_length", "128", "-max_tgt_length", "128",
           "-optim", "adam", "-learning_rate", "0.0005", "-update_method", "regular", "-weight_decay", "0.01", "-max_grad_norm", "5",
           "-label_smoothing", "0.1", "-dropout", "0.1", "-attn_dropout", "0.1", "-epochs", "100", "-max_step", str(args.updates),
           "-log_interval", str(every), "-save_every", "100000000", "-seed", "7"] + size
    if cuda:
        cmd += ["-fp16", "-bf16", "-gpus"] + [str(i) for i in range(args.gpus)]
    log_path = os.path.join(tmp, "train.log")
    env = dict(os.environ)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    with open(log_path, "w") as log:
        rc = subprocess.run(cmd, stdout=log, stderr=subprocess.STDOUT, env=env).returncode
    lines = [l for l in open(log_path) if "tgt tok/s" in l]
    rates = [float(m.group(1)) for l in lines for m in [re.search(r"([0-9.]+) tgt tok/s", l)] if m]
    steady = rates[len(rates) // 2:] if len(rates) >= 4 else rates     # shape classes are captured during the first epoch
    out = {"metric": "train target tokens/s through train_distributed.py", "unit": "tokens/s", "n_gpus": args.gpus if cuda else 0,
           "updates": args.updates, "exit_code": rc, "log_lines": len(rates),
           "value": float(np.median(steady)) if steady else None, "all_windows": rates,
           "config": {"model": "transformer-big 6+6 d1024 h16 ffn4096 relu vocab32000 tied" if not args.tiny else "tiny",
                      "batch_size_words": 13000 if not args.tiny else 300, "data": "synthetic corpus through preprocess.py"}}
    print(json.dumps(out), flush=True)
    if rc != 0:
        sys.stderr.write("".join(open(log_path).readlines()[-30:]))
        sys.exit(rc)


if __name__ == "__main__":
    main()
