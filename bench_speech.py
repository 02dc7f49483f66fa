"""Training throughput of the two speech configurations: Whisper-large-v2 and wav2vec2-large + mBART-50 decoder.

    python bench_speech.py --config whisper_large_v2|wav2vec2_mbart50 [--gpus N] [--steps K] [--warmup W] [--ddp fused|nccl|fsdp]
    python -m torch.distributed.run --nproc-per-node N ... bench_speech.py --gpus N ...        (N > 1)

Synthetic data of the real shapes and random-init weights of the real sizes (no checkpoint or corpus is reachable):

* ``whisper_large_v2``: 32 + 32 layers, d_model 1280, 20 heads, FFN 5120, 80 mel bins, 1500 encoder positions, vocabulary
  51865; every utterance is a 30 s window (3000 mel frames) with 60-200 target tokens.
* ``wav2vec2_mbart50``: wav2vec 2.0 large encoder on raw 16 kHz audio (7-layer convolutional front end, 24 layers,
  d_model 1024) + 12-layer mBART-50 style decoder, vocabulary 250054; utterances of 5-15 s with 20-80 target tokens.

Same timing rules as ``bench.py``: W warm-up steps, then K steps bracketed by a barrier + device synchronisation, CUDA
events, maximum over ranks; the value is the whole-job sum.  One JSON line on rank 0 with target tokens/s and audio
seconds/s.  ``--tiny`` shrinks both models for a CPU dry run.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import bench as B                                                             # noqa: E402  (timing helpers)


def _json(tmp, name, **kw):
    p = os.path.join(tmp, name)
    with open(p, "w") as fh:
        json.dump(kw, fh)
    return p


def build(config: str, tiny: bool, tmp: str):
    from nmtgminor_b200.data.synthetic import synthetic_audio_batch, synthetic_dict
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import default_options
    common = ["-dropout", "0.1", "-attn_dropout", "0.1", "-label_smoothing", "0.1", "-optim", "adam", "-weight_decay", "0.01",
              "-learning_rate", "0.0001", "-update_method", "regular", "-max_grad_norm", "1", "-fp16", "-bf16"]
    if config == "whisper_large_v2":
        dim, layers, heads, ffn, vocab, frames = (1280, 32, 20, 5120, 51865 // 8 * 8, 3000) if not tiny else (128, 2, 2, 256, 512, 200)
        cfg = _json(tmp, "whisper.json", d_model=dim, encoder_layers=layers, decoder_layers=layers, encoder_attention_heads=heads,
                    encoder_ffn_dim=ffn, num_mel_bins=80, max_source_positions=frames // 2, max_target_positions=448,
                    vocab_size=vocab, pad_token_id=0)
        opt = default_options(["-model", "whisper", "-dec_config_file", cfg, "-model_size", str(dim), "-n_heads", str(heads),
                               "-inner_size", str(ffn), "-layers", str(layers)] + common)
        n_utt = 8 if not tiny else 2
        make = lambda seed: synthetic_audio_batch(n_utt, vocab, "feats", n_feats=80, fixed_frames=frames, tgt_min=60 if not tiny else 5,
                                                  tgt_max=200 if not tiny else 12, seed=seed)
        seconds = lambda b: n_utt * frames / 100.0
        name = "whisper-large-v2 32+32 d1280 h20 ffn5120 vocab51865" if not tiny else "whisper (tiny dry run)"
    elif config == "wav2vec2_mbart50":
        dim, layers, heads, ffn, dec_layers, vocab = (1024, 24, 16, 4096, 12, 250054 // 8 * 8) if not tiny else (64, 2, 2, 128, 2, 512)
        enc = _json(tmp, "enc.json", encoder_embed_dim=dim, encoder_layers=layers, encoder_attention_heads=heads, encoder_ffn_embed_dim=ffn)
        dec = _json(tmp, "dec.json", d_model=dim, decoder_layers=dec_layers, decoder_attention_heads=heads, decoder_ffn_dim=ffn,
                    vocab_size=vocab, pad_token_id=0)
        opt = default_options(["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model", "mbart50",
                               "-model_size", str(dim), "-n_heads", str(heads), "-inner_size", str(ffn), "-layers", str(dec_layers)] + common)
        n_utt = 8 if not tiny else 2
        lo, hi = (80000, 240000) if not tiny else (3000, 6000)
        make = lambda seed: synthetic_audio_batch(n_utt, vocab, "wav", lo, hi, tgt_min=20 if not tiny else 5, tgt_max=80 if not tiny else 12,
                                                  seed=seed)
        seconds = lambda b: float(b.get("src_lengths").sum()) / 16000.0
        name = "wav2vec2-large + mbart50 decoder 24+12 d1024 vocab250054" if not tiny else "wav2vec2 + mbart50 (tiny dry run)"
    else:
        raise SystemExit("unknown --config %r" % config)
    d = synthetic_dict(vocab)
    model = build_model(opt, {"src": d, "tgt": d})
    return opt, model, make, seconds, name


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="whisper_large_v2", choices=["whisper_large_v2", "wav2vec2_mbart50"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ddp", default="fused", choices=["fused", "nccl", "fsdp"])
    ap.add_argument("--tiny", action="store_true", help="small models (CPU dry run)")
    args = ap.parse_args(argv)
    from nmtgminor_b200.train.engine import TrainEngine
    cuda = torch.cuda.is_available()
    rank, local, world = B.dist_setup(args.gpus) if cuda else (0, 0, 1)
    torch.manual_seed(4321)
    with tempfile.TemporaryDirectory() as tmp:
        opt, model, make, seconds, name = build(args.config, args.tiny, tmp)
    n_params = sum(p.numel() for p in model.parameters())
    engine = TrainEngine(model, opt, device=("cuda:%d" % local) if cuda else "cpu", cuda_graph=False,
                         ddp=(args.ddp if (world > 1 or args.ddp == "fsdp") else None))
    batches = [make(100 * rank + i) for i in range(4)]
    if cuda:
        batches = [b.pin_memory() for b in batches]
    tokens = [b.tgt_size for b in batches]
    secs = [seconds(b) for b in batches]
    step = lambda b: engine.train_step(b)[0]
    loss = None
    for i in range(args.warmup):
        loss = step(batches[i % len(batches)])
    first_loss = float(loss) / tokens[(args.warmup - 1) % len(batches)] if args.warmup else None
    if cuda:
        ms, ntok = B.timed_loop(step, batches, tokens, args.steps, world, read_loss=True)
        peak0 = torch.cuda.max_memory_allocated() / 2 ** 30
        total_tok = B.sum_over_ranks(float(ntok), world)
        audio = B.sum_over_ranks(float(sum(secs[i % len(secs)] for i in range(args.steps))), world)
        from nmtgminor_b200 import ops
        status = ops.check_status()
    else:
        import time
        t0 = time.time()
        ntok = 0
        for i in range(args.steps):
            float(step(batches[i % len(batches)]))
            ntok += tokens[i % len(batches)]
        ms, total_tok, audio, status, peak0 = (time.time() - t0) * 1e3, float(ntok), float(sum(secs[i % len(secs)] for i in range(args.steps))), 0, 0.0
    if rank == 0:
        print(json.dumps({
            "metric": "train target tokens/s", "value": total_tok / (ms / 1e3), "unit": "tokens/s",
            "audio_seconds_per_second": audio / (ms / 1e3), "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic", "impl": "ours",
            "config": {"model": name, "params": n_params, "utterances_per_gpu": len(batches[0].get("src_lengths")),
                       "parallelism": "dp%d" % world, "ddp": args.ddp if (world > 1 or args.ddp == "fsdp") else None,
                       "timing": "end to end: pinned host batch -> device and loss read back every step"},
            "peak_memory_gib": peak0, "kernel_status": status, "loss_per_token_after_warmup": first_loss}), flush=True)
    if world > 1 and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
