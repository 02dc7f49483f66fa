"""Training throughput of the two speech configurations: Whisper-large-v2 and wav2vec2-large + mBART-50 decoder.

    python bench_speech.py --config whisper_large_v2|wav2vec2_mbart50 [--gpus N] [--steps K] [--warmup W] [--ddp fused|nccl|fsdp]
    python -m torch.distributed.run --nproc-per-node N ... bench_speech.py --gpus N ...        (N > 1)

Synthetic data of the real shapes and random-init weights of the real sizes (no checkpoint or corpus is reachable):

* ``whisper_large_v2``: 32 + 32 layers, d_model 1280, 20 heads, FFN 5120, 80 mel bins, 1500 encoder positions, vocabulary
  51865; 16 utterances per GPU, each a 30 s window (80 x 3000 log-mel frames ~ N(0, 1)) with 20-448 target tokens;
  fully sharded parameters by default (``--ddp fsdp``), AdamW.
* ``wav2vec2_mbart50``: wav2vec 2.0 large encoder on raw 16 kHz audio ~ N(0, 0.1) (7-layer convolutional front end, 24
  layers, d_model 1024) + 12-layer mBART-50 style decoder, vocabulary 250054; utterances of 5-20 s, about 1.2 M samples
  per GPU batch, 10-120 target tokens.

``--impl reference`` runs the unmodified reference on the same shapes (``bench_speech_reference.py``): its Hugging Face
path model ``MemoryEfficientWhisper`` under torch FSDP for Whisper; for wav2vec2 + mBART it prints ``unavailable``
(the reference's wrapper needs the ``omegaconf`` package, which is not installed and not in the wheelhouse).

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


def build(config: str, tiny: bool, tmp: str, want_model: bool = True):
    from nmtgminor_b200.data.synthetic import synthetic_audio_batch, synthetic_dict
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import default_options
    common = ["-dropout", "0.1", "-attn_dropout", "0.1", "-label_smoothing", "0.1", "-optim", "adam", "-weight_decay", "0.01",
              "-learning_rate", "0.0001", "-update_method", "regular", "-max_grad_norm", "1", "-fp16", "-bf16"]
    if config == "whisper_large_v2":
        dim, layers, heads, ffn, vocab, frames = (1280, 32, 20, 5120, 51865, 3000) if not tiny else (128, 2, 2, 256, 517, 200)
        cfg = _json(tmp, "whisper.json", d_model=dim, encoder_layers=layers, decoder_layers=layers, encoder_attention_heads=heads,
                    encoder_ffn_dim=ffn, num_mel_bins=80, max_source_positions=frames // 2, max_target_positions=448,
                    vocab_size=vocab, pad_token_id=0)
        opt = default_options(["-model", "whisper", "-dec_config_file", cfg, "-model_size", str(dim), "-n_heads", str(heads),
                               "-inner_size", str(ffn), "-layers", str(layers)] + common)
        n_utt = 16 if not tiny else 2
        # 20-448 target tokens counting the start and end symbols (448 is the decoder's last position)
        make = lambda seed: synthetic_audio_batch(n_utt, vocab, "feats", n_feats=80, fixed_frames=frames, tgt_min=18 if not tiny else 5,
                                                  tgt_max=446 if not tiny else 12, seed=seed)
        seconds = lambda b: n_utt * frames / 100.0
        name = "whisper-large-v2 32+32 d1280 h20 ffn5120 vocab51865" if not tiny else "whisper (tiny dry run)"
    elif config == "wav2vec2_mbart50":
        dim, layers, heads, ffn, dec_layers, vocab = (1024, 24, 16, 4096, 12, 250054) if not tiny else (64, 2, 2, 128, 2, 518)
        enc = _json(tmp, "enc.json", encoder_embed_dim=dim, encoder_layers=layers, encoder_attention_heads=heads, encoder_ffn_embed_dim=ffn)
        dec = _json(tmp, "dec.json", d_model=dim, decoder_layers=dec_layers, decoder_attention_heads=heads, decoder_ffn_dim=ffn,
                    vocab_size=vocab, pad_token_id=0)
        opt = default_options(["-model", "wav2vec2_bert", "-enc_config_file", enc, "-dec_config_file", dec, "-dec_pretrained_model", "mbart50",
                               "-model_size", str(dim), "-n_heads", str(heads), "-inner_size", str(ffn), "-layers", str(dec_layers)] + common)
        n_utt = 6 if not tiny else 2               # 6 utterances of 5-20 s (12.5 s on average) = 1.2 M samples per batch
        lo, hi = (80000, 320000) if not tiny else (3000, 6000)
        make = lambda seed: synthetic_audio_batch(n_utt, vocab, "wav", lo, hi, tgt_min=10 if not tiny else 5, tgt_max=120 if not tiny else 12,
                                                  seed=seed)
        seconds = lambda b: float(b.get("src_lengths").sum()) / 16000.0
        name = "wav2vec2-large + mbart50 decoder 24+12 d1024 vocab250054" if not tiny else "wav2vec2 + mbart50 (tiny dry run)"
    else:
        raise SystemExit("unknown --config %r" % config)
    sizes = dict(dim=dim, layers=layers, heads=heads, ffn=ffn, vocab=vocab, n_mels=80, frames=frames if config == "whisper_large_v2" else 0)
    if not want_model:
        return opt, None, make, seconds, name, sizes
    d = synthetic_dict(vocab)
    model = build_model(opt, {"src": d, "tgt": d})
    return opt, model, make, seconds, name, sizes


def run_reference(args):
    """The reference arm on the same batches (see ``bench_speech_reference.py``)."""
    cuda = torch.cuda.is_available()
    if args.config != "whisper_large_v2":
        print(json.dumps({"impl": "reference", "unavailable": "the reference's wav2vec 2.0 wrapper imports omegaconf (OmegaConf.create / "
                          "set_struct on the checkpoint's cfg, onmt/models/speech_recognizer/wav2vec2.py:11,79-81), which is neither "
                          "installed nor in the offline wheelhouse"}), flush=True)
        return
    rank, local, world = B.dist_setup(args.gpus) if cuda else (0, 0, 1)
    torch.manual_seed(4321)
    with tempfile.TemporaryDirectory() as tmp:
        _opt, _none, make, seconds, name, sizes = build(args.config, args.tiny, tmp, want_model=False)
    try:
        from bench_speech_reference import WhisperReferenceRunner
        runner = WhisperReferenceRunner(sizes, ("cuda:%d" % local) if cuda else "cpu", rank, world)
    except Exception as exc:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference's Whisper model did not build: %r" % (exc,)}), flush=True)
        return
    ours = [make(100 * rank + i) for i in range(4)]
    batches, tokens, secs = [], [], []
    for b in ours:                           # the same utterances and targets, in the reference's input layout
        src = b.get("source")                # [T, B, 1 + n_mels]: channel 0 marks real frames
        feats = [src[:, i, 1:] for i in range(src.shape[1])]
        tgt = b.get("target")                # [T, B] with BOS ... EOS, 0 = padding
        lens = b.get("tgt_lengths").tolist()
        targets = [tgt[:n, i] for i, n in enumerate(lens)]
        batches.append(runner.collate(feats, targets))
        tokens.append(batches[-1][2])
        secs.append(seconds(b))
    step = runner.step
    for i in range(args.warmup):
        step(batches[i % len(batches)])
    if cuda:
        torch.cuda.reset_peak_memory_stats()
        ms, ntok = B.timed_loop(step, batches, tokens, args.steps, world, read_loss=True)
        peak = torch.cuda.max_memory_allocated() / 2 ** 30
        total_tok = B.sum_over_ranks(float(ntok), world)
        audio = B.sum_over_ranks(float(sum(secs[i % len(secs)] for i in range(args.steps))), world)
    else:
        import time
        t0 = time.time()
        ntok = 0
        for i in range(args.steps):
            float(step(batches[i % len(batches)]))
            ntok += tokens[i % len(batches)]
        ms, total_tok, audio, peak = (time.time() - t0) * 1e3, float(ntok), float(sum(secs[i % len(secs)] for i in range(args.steps))), 0.0
    if rank == 0:
        print(json.dumps({
            "metric": "train target tokens/s", "value": total_tok / (ms / 1e3), "unit": "tokens/s",
            "audio_seconds_per_second": audio / (ms / 1e3), "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic", "impl": "reference",
            "config": {"model": name, "params": runner.n_params, "utterances_per_gpu": len(ours[0].get("src_lengths")),
                       "parallelism": "dp%d" % world, "timing": "end to end: pinned host batch -> device and loss read back every step"},
            "impl_details": {"path": runner.path}, "peak_memory_gib": peak}), flush=True)
    if world > 1 and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="whisper_large_v2", choices=["whisper_large_v2", "wav2vec2_mbart50"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ddp", default=None, choices=["fused", "nccl", "fsdp"],
                    help="default: fsdp for whisper_large_v2 (the configuration names it), fused otherwise")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tiny", action="store_true", help="small models (CPU dry run)")
    args = ap.parse_args(argv)
    if args.ddp is None:
        args.ddp = "fsdp" if args.config == "whisper_large_v2" else "fused"
    if args.impl == "reference":
        return run_reference(args)
    from nmtgminor_b200.train.engine import TrainEngine
    cuda = torch.cuda.is_available()
    rank, local, world = B.dist_setup(args.gpus) if cuda else (0, 0, 1)
    torch.manual_seed(4321)
    with tempfile.TemporaryDirectory() as tmp:
        opt, model, make, seconds, name, _sizes = build(args.config, args.tiny, tmp)
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
                       "parallelism": "dp%d" % world, "timing": "end to end: pinned host batch -> device and loss read back every step"},
            "impl_details": {"ddp": args.ddp if (world > 1 or args.ddp == "fsdp") else None,
                             "memory_report": engine.optim.distributed.memory_report() if hasattr(getattr(engine.optim, "distributed", None), "memory_report") else None},
            "peak_memory_gib": peak0, "kernel_status": status, "loss_per_token_after_warmup": first_loss}), flush=True)
    if world > 1 and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
