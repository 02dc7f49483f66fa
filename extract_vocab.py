#!/usr/bin/env python
"""python extract_vocab.py -dict data.dict.pt -text "a.txt|b.txt" [-external_tokenizer <name or dir>] [-lang en_XX]
       [-input_type word|char] -output used_ids.pt
Counts which vocabulary ids occur in the given text files (to shrink an output layer to the ids a task uses) and saves
``{id: count}`` sorted by count.  (reference: extract_vocab.py)"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-dict", required=True, help="dictionary file written by preprocess.py (a dict of Dicts, one Dict, or a raw-format data file)")
    ap.add_argument("-text", required=True, help="text files separated by |")
    ap.add_argument("-external_tokenizer", default="")
    ap.add_argument("-lang", default="")
    ap.add_argument("-input_type", default="word", choices=["word", "char"])
    ap.add_argument("-output", default="pred.txt")
    opt = ap.parse_args(argv)
    dictionary = torch.load(opt.dict, weights_only=False)
    if isinstance(dictionary, dict):
        dictionary = dictionary.get("dicts", dictionary)          # a raw-format data file carries its dictionaries
        dictionary = dictionary.get("tgt") or dictionary.get("src")
    external = None
    if opt.external_tokenizer:
        from nmtgminor_b200.data.binarizer import load_external_tokenizer
        external = load_external_tokenizer(opt.external_tokenizer, opt.lang or None)
    counts = {}
    unk = dictionary.lookup("<unk>") if dictionary is not None else 0
    for path in opt.text.split("|"):
        print("Loading from data %s ..." % path)
        with open(path) as fh:
            for line in fh:
                if external is not None:
                    ids = external(line.strip())
                else:
                    toks = line.split() if opt.input_type == "word" else list(line.strip())
                    ids = [dictionary.lookup(t, unk) for t in toks]
                for i in ids:
                    i = int(i)
                    counts[i] = counts.get(i, 0) + 1
    counts = dict(sorted(counts.items(), key=lambda kv: kv[1]))
    print("saving %d ids to %s" % (len(counts), opt.output))
    torch.save(counts, opt.output)


if __name__ == "__main__":
    main()
