#!/usr/bin/env python
"""Beam-search throughput (generated target tokens per second) of Transformer-big with random weights.

    python bench_translate.py [--batch 64] [--beam 4] [--src-len 30] [--max-len 40] [--steps 5] [--warmup 2] [--plain]

Every step translates one synthetic batch end to end (encoder, incremental decoder, beam search, hypotheses on the
host).  ``min_len == max_len`` makes every hypothesis exactly ``max_len`` tokens long, so the amount of work does not
depend on the random weights.  Prints one JSON line.
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--beam", type=int, default=4)
    ap.add_argument("--src-len", type=int, default=30)
    ap.add_argument("--max-len", type=int, default=40)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--plain", action="store_true", help="PyTorch log-softmax / top-k instead of the fused beam kernel")
    ap.add_argument("--no-graph", action="store_true", help="launch the decoding step kernel by kernel instead of replaying CUDA graphs")
    args = ap.parse_args()

    from nmtgminor_b200 import ops
    from nmtgminor_b200.data.dataset import collate
    from nmtgminor_b200.data.synthetic import synthetic_dict
    from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search
    from nmtgminor_b200.models.transformer import Transformer
    from nmtgminor_b200.options import default_options
    from nmtgminor_b200.parallel.flat import FlatParameterStore

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    d = synthetic_dict(args.vocab)
    opt = default_options(["-model_size", "1024", "-layers", "6", "-n_heads", "16", "-inner_size", "4096", "-tie_weights",
                           "-join_embedding", "-ffn_activation", "relu"])
    model = Transformer(opt, {"src": d, "tgt": d}).eval()
    FlatParameterStore(model, dev)
    for b in model.buffers():
        b.data = b.data.to(dev)
    model.renew_buffer(max(args.src_len, args.max_len) + 4)
    g = torch.Generator().manual_seed(1)
    cfg = BeamConfig(beam_size=args.beam, n_best=1, max_len=args.max_len, min_len=args.max_len, fused_step=not args.plain,
                     cuda_graph=not args.no_graph)

    def one():
        src = [torch.randint(4, args.vocab, (args.src_len,), generator=g) for _ in range(args.batch)]
        batch = collate(src, None, padded=True, packed=True, round_to=1).cuda(dev)
        hyps = beam_search(model, batch, cfg)
        return sum(len(h[0].tokens) for h in hyps)

    for _ in range(args.warmup):
        one()
    torch.cuda.synchronize()
    ops.LAUNCHES[0] = 0
    t0 = time.perf_counter()
    toks = 0
    for _ in range(args.steps):
        toks += one()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    print(json.dumps({"metric": "beam_search_generated_tokens_per_second", "value": toks / dt, "unit": "tokens/s",
                      "ms_per_batch": 1e3 * dt / args.steps, "ms_per_decode_step": 1e3 * dt / args.steps / (args.max_len + 1),
                      "tokens": toks, "gpu_launches": ops.LAUNCHES[0], "status": ops.check_status(),
                      "config": {"model": "transformer-big", "batch": args.batch, "beam": args.beam, "src_len": args.src_len,
                                 "max_len": args.max_len, "vocab": args.vocab, "fused_step": not args.plain, "cuda_graph": not (args.no_graph or args.plain)},
                      "dtype": "bf16", "data": "synthetic"}))


if __name__ == "__main__":
    main()
