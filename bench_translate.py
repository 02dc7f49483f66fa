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


def run_reference(args):
    """The unmodified reference's ``FastTranslator`` on the same model size and batch geometry (a checkpoint with
    random weights is written in the reference's own format and loaded through its public API)."""
    import tempfile
    os.environ.setdefault("TORCH_FORCE_NO_WEIGHTS_ONLY_LOAD", "1")      # the reference calls torch.load() on a pickled Namespace
    import bench_reference as br
    from nmtgminor_b200.options import make_translate_parser
    if not br.reference_available():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    # The reference's beam search writes the Whisper prompt ids (50258, 50265, 50360, 50364) into the first four target
    # positions of every hypothesis and starts decoding at step 3 whatever the model is
    # (onmt/inference/fast_translator.py:462-469, :661).  Smaller vocabularies would index past the embedding table, so
    # the reference arm only runs with a vocabulary that contains those ids; it then performs max_len - 2 decoder steps.
    # With a large enough vocabulary the first decoder call then receives four target positions while the Transformer's
    # incremental step builds its masks for one (onmt/modules/attention.py:126 raises "output with shape [.., 1, 1] doesn't
    # match the broadcast shape [.., 1, 4]"), so the stock translator cannot decode a text Transformer at all.  The arm is
    # reported as unavailable; --force-reference runs it anyway on the CPU to show the error.  The reference's other search,
    # Translator.translate_batch (onmt/inference/translator.py:331, one Beam object per sentence), was tried on the CPU as
    # well and stops at the same line ("output with shape [1, 4, 1, 1] doesn't match the broadcast shape [1, 4, 1, 32]").
    if not args.force_reference or torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "the reference's FastTranslator hard-codes the Whisper prompt "
                          "(token ids up to 50364, decoding from step 3); it and the legacy Translator.translate_batch both fail in the "
                          "Transformer's incremental attention mask (onmt/modules/attention.py:126: output with shape [1, 4, 1, 1] "
                          "doesn't match the broadcast shape [1, 4, 1, 32])"}))
        return
    cuda = torch.cuda.is_available()
    runner = br.ReferenceRunner(args.vocab, "cuda:0" if cuda else "cpu", tiny=args.tiny)
    onmt = runner.onmt
    d = onmt.Dict(["<blank>", "<unk>", "<s>", "</s>"])
    for i in range(args.vocab - 4):
        d.add("w%d" % i)
    dicts = {"src": d, "tgt": d, "langs": {"src": 0, "tgt": 1}, "atbs": {"nothingness": 0}}
    tmp = tempfile.NamedTemporaryFile(suffix=".pt", delete=False)
    torch.save({"model": runner.raw_model.state_dict(), "dicts": dicts, "opt": runner.opt, "epoch": 1, "optim": None}, tmp.name)
    del runner
    topt = make_translate_parser().parse_args(["-model", tmp.name, "-src", "none", "-beam_size", str(args.beam), "-batch_size", str(args.batch),
                                               "-max_sent_length", str(args.max_len), "-min_sent_length", str(args.max_len)])
    topt.cuda = cuda
    topt.gpu = 0 if cuda else -1
    topt.fp16, topt.bf16 = False, cuda
    topt.verbose = False
    topt.fast_translate = True
    if cuda:
        torch.cuda.set_device(0)
    from onmt.inference.fast_translator import FastTranslator
    translator = FastTranslator(topt)
    g = torch.Generator().manual_seed(1)

    def one():
        src = [["w%d" % int(t) for t in torch.randint(0, args.vocab - 4, (args.src_len,), generator=g)] for _ in range(args.batch)]
        out = translator.translate(src, None)
        return sum(len(p[0]) for p in out[0])

    for _ in range(args.warmup):
        one()
    if cuda:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    toks = sum(one() for _ in range(args.steps))
    if cuda:
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    os.unlink(tmp.name)
    print(json.dumps({"impl": "reference", "metric": "beam_search_generated_tokens_per_second", "value": toks / dt, "unit": "tokens/s",
                      "ms_per_batch": 1e3 * dt / args.steps, "ms_per_decode_step": 1e3 * dt / args.steps / max(args.max_len - 2, 1),
                      "decode_steps_per_batch": args.max_len - 2, "tokens": toks,
                      "config": {"model": "transformer-big" if not args.tiny else "tiny", "batch": args.batch, "beam": args.beam,
                                 "src_len": args.src_len, "max_len": args.max_len, "vocab": args.vocab},
                      "dtype": "bf16" if cuda else "fp32", "data": "synthetic"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tiny", action="store_true", help="reference arm only: small model (for a CPU dry run)")
    ap.add_argument("--force-reference", action="store_true", help="reference arm: attempt the run on the CPU although it is known to fail")
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
    if args.impl == "reference":
        return run_reference(args)

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
