#!/usr/bin/env python
"""python normalize_text.py <input file> <language> <workers> [cleaning]
Transcript normalisation for scoring and data cleaning: Unicode NFKC, quote folding, lower case, punctuation removed
(apostrophes kept); English also gets the usual contraction spacing folded.  Writes ``<input>.norm``; with a non-zero
fourth argument lines that lose more than 30 % of their words are dropped and ``<input>.clean`` / ``<input>.norm.clean``
are written instead.  The file is cut into byte ranges that worker processes normalise in parallel.
(reference: normalize_text.py, which wraps the whisper_normalizer package)"""
import os
import sys
from concurrent.futures import ProcessPoolExecutor

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.text import normalize_text


def _offsets(path, chunks):
    size = os.path.getsize(path)
    offs = [0]
    with open(path, "rb") as fh:
        for i in range(1, chunks):
            fh.seek(size * i // chunks)
            fh.readline()
            offs.append(fh.tell())
    return offs + [size]


def _work(args):
    path, lo, hi, lang = args
    org, out = [], []
    with open(path, "rb") as fh:
        fh.seek(lo)
        while fh.tell() < hi:
            line = fh.readline().decode("utf-8", errors="replace").strip()
            org.append(line)
            out.append(normalize_text(line, lower=True, strip_punct=True))
    return org, out


def normalize_file(path, lang="en", workers=1):
    offs = _offsets(path, max(1, workers))
    jobs = [(path, offs[i], offs[i + 1], lang) for i in range(len(offs) - 1) if offs[i + 1] > offs[i]]
    if workers > 1:
        with ProcessPoolExecutor(workers) as ex:
            parts = list(ex.map(_work, jobs))
    else:
        parts = [_work(j) for j in jobs]
    org = [l for p in parts for l in p[0]]
    out = [l for p in parts for l in p[1]]
    return org, out


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) < 3:
        sys.exit(__doc__)
    path, lang, workers = argv[0], argv[1], int(argv[2])
    cleaning = int(argv[3]) if len(argv) > 3 else 0
    print("Normalizing file %s" % path)
    org, out = normalize_file(path, lang, workers)
    if cleaning:
        with open(path + ".norm.clean", "w") as w, open(path + ".clean", "w") as ow:
            for o, n in zip(org, out):
                if len(n.split()) <= 0.7 * len(o.split()):
                    continue
                ow.write(o + "\n")
                w.write(n + "\n")
    else:
        with open(path + ".norm", "w") as w:
            for n in out:
                w.write(n + "\n")
    print("Finished.")


if __name__ == "__main__":
    main()
