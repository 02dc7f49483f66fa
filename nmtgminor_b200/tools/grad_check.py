"""Finite-difference gradient check of the reversible encoder / decoder stacks in float64.

    python -m nmtgminor_b200.tools.grad_check [-model_size 16] [-layers 2] [-test_decoder] [-gpu -1]

The reversible stacks carry a hand-written backward (inputs are reconstructed from the outputs, the sub-layers are
replayed), so their gradients are checked numerically against central differences, for the input states and, for the
decoder, the encoder memory.  (reference: tools/grad_check.py:31-99, tools/grad_check_reversible.py)"""
from __future__ import annotations

import argparse

import torch

from ..models.layers import PackedSeqs
from ..models.reversible import ReversibleStack


def packed(lengths, device="cpu") -> PackedSeqs:
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    pos = torch.cat([torch.arange(l) for l in lengths])
    return PackedSeqs(torch.zeros(int(cu[-1]), dtype=torch.long, device=device), pos.to(device), cu.to(device), max(lengths))


def check_reversible(model_size: int = 16, layers: int = 2, heads: int = 1, decoder: bool = False, device="cpu",
                     lengths=(5, 3), mem_lengths=(4, 2), seed: int = 0) -> bool:
    """``torch.autograd.gradcheck`` of a reversible stack without dropout; raises if a gradient is off."""
    torch.manual_seed(seed)
    seqs = packed(list(lengths), device)
    stack = ReversibleStack(layers, model_size, heads, model_size, dropout=0.0, attn_dropout=0.0, causal=decoder,
                            cross=decoder).double().to(device).train()
    x = torch.randn(int(seqs.cu[-1]), model_size, dtype=torch.float64, device=device, requires_grad=True)
    if not decoder:
        return torch.autograd.gradcheck(lambda a: stack(a, seqs), (x,), eps=1e-6, atol=1e-5, rtol=1e-4)
    mem_seqs = packed(list(mem_lengths), device)
    mem = torch.randn(int(mem_seqs.cu[-1]), model_size, dtype=torch.float64, device=device, requires_grad=True)
    return torch.autograd.gradcheck(lambda a, m: stack(a, seqs, m, mem_seqs), (x, mem), eps=1e-6, atol=1e-5, rtol=1e-4)


def main(argv=None):
    ap = argparse.ArgumentParser(description="gradient check of the reversible Transformer stacks")
    ap.add_argument("-model_size", type=int, default=16)
    ap.add_argument("-layers", type=int, default=2)
    ap.add_argument("-n_heads", type=int, default=1)
    ap.add_argument("-gpu", type=int, default=-1)
    ap.add_argument("-test_decoder", action="store_true")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", a.gpu) if a.gpu >= 0 and torch.cuda.is_available() else torch.device("cpu")
    print("start gradchecking the %s ..." % ("decoder (input and context)" if a.test_decoder else "encoder"))
    check_reversible(a.model_size, a.layers, a.n_heads, a.test_decoder, dev)
    print("gradchecking completed.")


if __name__ == "__main__":
    main()
