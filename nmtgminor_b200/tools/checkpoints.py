"""Checkpoint utilities: averaging (arithmetic / geometric), picking the best files by the metric in their names,
growing the vocabulary of a trained model, and re-matching embeddings by token string between two dictionaries.

Command line:  python -m nmtgminor_b200.tools.checkpoints average -models a.pt b.pt -output avg.pt [-method mean|gmean]
               python -m nmtgminor_b200.tools.checkpoints best -prefix model -top 5
Reference: tools/average_checkpoints.py:25-115, average_checkpoints_auto.py, extend_weight.py,
tools/extend_deltalm_vocab.py, rematch_language_embedding.py, onmt/train_utils/mp_trainer.py:438-510.
"""
from __future__ import annotations

import argparse
import glob
import re
from typing import Dict, List

import torch


def average_state_dicts(states: List[Dict[str, torch.Tensor]], method: str = "mean") -> Dict[str, torch.Tensor]:
    out = {}
    for k in states[0]:
        vals = [s[k].double() for s in states if k in s]
        if not vals[0].is_floating_point() and not torch.is_floating_point(states[0][k]):
            out[k] = states[0][k].clone()
            continue
        if method == "gmean":
            sign = torch.sign(sum(vals))
            mag = torch.exp(sum(torch.log(v.abs().clamp_min(1e-30)) for v in vals) / len(vals))
            out[k] = (sign * mag).to(states[0][k].dtype)
        else:
            out[k] = (sum(vals) / len(vals)).to(states[0][k].dtype)
    return out


def average_checkpoints(paths: List[str], output: str, method: str = "mean"):
    ckpts = [torch.load(p, map_location="cpu", weights_only=False) for p in paths]
    base = ckpts[0]
    base["model"] = average_state_dicts([c["model"] for c in ckpts], method)
    base["optim"] = None
    torch.save(base, output)
    return output


def best_checkpoints(prefix: str, top: int = 5, metric: str = "ppl", lower_is_better: bool = True) -> List[str]:
    scored = []
    for f in glob.glob(glob.escape(prefix) + "_" + metric + "_*_e*.pt"):
        m = re.search(r"_%s_([-0-9.eE+]+)_e([0-9.]+)\.pt$" % metric, f)
        if m:
            scored.append((float(m.group(1)), f))
    scored.sort(reverse=not lower_is_better)
    return [f for _, f in scored[:top]]


def extend_vocabulary(state: Dict[str, torch.Tensor], keys: List[str], new_size: int, init_std: float = 0.02):
    """Grow the first dimension of the named tensors (embeddings / output layer) to ``new_size`` rows."""
    for k in keys:
        w = state[k]
        if w.shape[0] >= new_size:
            continue
        extra = torch.zeros((new_size - w.shape[0],) + tuple(w.shape[1:]), dtype=w.dtype)
        if w.dim() > 1:
            extra.normal_(0, init_std)
        state[k] = torch.cat([w, extra], 0)
    return state


def extend_pretrained_vocab(weights: Dict[str, torch.Tensor], keys: List[str], base_size: int, extra: int, seed: int = 0):
    """Embedding tables of a pre-trained model (DeltaLM, mBART) grown for ``extra`` new symbols, e.g. speech units: the
    first ``base_size`` rows are kept (rows past them, the pre-training mask tokens, are dropped) and every new row
    starts as a copy of a randomly chosen kept row, so that it lies inside the distribution the model was trained
    with.  (reference: tools/extend_deltalm_vocab.py:17-72)"""
    gen = torch.Generator().manual_seed(seed)
    for k in keys:
        if k not in weights:
            continue
        w = weights[k]
        if w.shape[0] < base_size:
            raise ValueError("%s has %d rows, fewer than the base vocabulary of %d" % (k, w.shape[0], base_size))
        picks = torch.randint(0, base_size, (extra,), generator=gen)
        weights[k] = torch.cat([w[:base_size], w[:base_size].index_select(0, picks)], 0).contiguous()
    return weights


def extend_vocab_file(path: str, extra: int, output: str = "") -> str:
    """Appends ``__0__ .. __<extra-1>__`` with the next free ids to a ``<token> <id>`` vocabulary file."""
    output = output or path + ".extend"
    with open(path) as fh:
        lines = fh.readlines()
    with open(output, "w") as out:
        out.writelines(l if l.endswith("\n") else l + "\n" for l in lines)
        for i in range(extra):
            out.write("__%d__ %d\n" % (i, len(lines) + i))
    return output


def rematch_embeddings(weight_old: torch.Tensor, dict_old, dict_new, init: torch.Tensor = None) -> torch.Tensor:
    """Rows of ``weight_old`` are copied to the ids the same token strings have in ``dict_new``."""
    out = init.clone() if init is not None else torch.zeros(dict_new.size(), weight_old.shape[1], dtype=weight_old.dtype).normal_(0, 0.02)
    copied = 0
    for idx in range(dict_new.size()):
        old = dict_old.lookup(dict_new.get_label(idx))
        if old is not None and old < weight_old.shape[0]:
            out[idx] = weight_old[old]
            copied += 1
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("average")
    a.add_argument("-models", nargs="+", required=True)
    a.add_argument("-output", required=True)
    a.add_argument("-method", default="mean", choices=["mean", "gmean"])
    b = sub.add_parser("best")
    b.add_argument("-prefix", required=True)
    b.add_argument("-top", type=int, default=5)
    b.add_argument("-output", default="")
    c = sub.add_parser("extend-vocab", help="grow the embedding tables of a pre-trained checkpoint for new symbols")
    c.add_argument("-input", required=True, help="checkpoint with its tensors under 'weights', 'model' or at the top level")
    c.add_argument("-vocab", required=True, help="'<token> <id>' vocabulary file")
    c.add_argument("-extra", type=int, default=5946, help="number of new symbols (e.g. k-means units)")
    c.add_argument("-base_size", type=int, default=250054)
    c.add_argument("-keys", nargs="+", default=["tgt_embedding.embed_tokens.weight", "src_embedding.embed_tokens.weight"])
    args = ap.parse_args(argv)
    if args.cmd == "extend-vocab":
        ckpt = torch.load(args.input, map_location="cpu", weights_only=False)
        holder = ckpt["weights"] if "weights" in ckpt else ckpt["model"] if "model" in ckpt else ckpt
        extend_pretrained_vocab(holder, args.keys, args.base_size, args.extra)
        torch.save(ckpt, args.input + ".extend")
        print(args.input + ".extend", extend_vocab_file(args.vocab, args.extra))
        return
    if args.cmd == "average":
        print(average_checkpoints(args.models, args.output, args.method))
    else:
        files = best_checkpoints(args.prefix, args.top)
        print("\n".join(files))
        if args.output and files:
            average_checkpoints(files, args.output)


if __name__ == "__main__":
    main()
