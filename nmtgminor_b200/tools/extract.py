"""Dump frame-level features of a wav2vec 2.0 style encoder for a list of recordings, the way Kaldi stores filterbank
features, so that any pipeline that reads ``ark`` / ``scp`` can train on them:

* ``extract_tdnn``     - output of the convolutional feature extractor (the "TDNN" front end, 512 channels at 20 ms),
                         or, with ``layer = n``, the states after ``n`` Transformer layers;
* ``extract_codes``    - product-quantiser code indices per frame (one line of ``group0:group1 ...`` pairs per utterance)
                         for encoders that carry a quantiser; with a k-means model the cluster of every frame instead.

The recordings come as a Kaldi-style list ``<utt> <wav path> [<start s> <end s>]``.  The model is either a checkpoint of
this framework whose encoder is a wav2vec 2.0 / HuBERT / WavLM encoder, or a fairseq pre-training checkpoint
(``{'cfg' | 'args', 'model'}``), whose architecture fields size the encoder.

Reference: extract_wav2vec2_tdnn.py:100-217 (batching by total samples, ark / scp writer), extract_wav2vec2_codebook.py:100-223,
onmt/models/speech_recognizer/wav2vec2.py (``FairseqWav2VecExtractor``, ``FairseqWav2VecQuantizer``).
"""
from __future__ import annotations

import os
from typing import Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..data.audio import read_ark_matrix, read_scp, read_wav, write_ark_matrix


def read_wav_list(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (utterance id, waveform [samples] float32) for every line of a ``<utt> <wav> [<start> <end>]`` file."""
    with open(path) as fh:
        for line in fh:
            parts = line.split()
            if not parts:
                continue
            start, end = (float(parts[2]), float(parts[3])) if len(parts) >= 4 else (0.0, 0.0)
            samples, _ = read_wav(parts[1], start, end)
            yield parts[0], torch.from_numpy(np.asarray(samples, dtype=np.float32)).reshape(-1)


def load_speech_encoder(path: str, device="cpu"):
    """The speech encoder of a checkpoint.  Returns (encoder module, quantiser module or None)."""
    state = torch.load(path, map_location="cpu", weights_only=False)
    if isinstance(state, dict) and "dicts" in state and "opt" in state:
        from ..models.factory import build_model
        from ..options import backward_compatible
        from ..train.checkpoint import load_model_state
        model = build_model(backward_compatible(state["opt"]), state["dicts"], remove_pretrain=True)
        load_model_state(model, state["model"])
        enc = model.encoder
    else:
        from ..models.pretrained_io import load_wav2vec2_checkpoint
        from ..models.speech_encoders import Wav2Vec2Encoder
        c = state.get("cfg") or state.get("args") or {}
        c = c.get("model", c) if isinstance(c, dict) else vars(c)
        g = lambda k, d: c.get(k, d) if isinstance(c, dict) else d
        conv = g("conv_feature_layers", None)
        kw = {}
        if isinstance(conv, str):
            kw["conv_layers"] = [tuple(x) for x in eval(conv, {"__builtins__": {}})]    # "[(512, 10, 5)] + [(512, 3, 2)] * 4 + ..."
        enc = Wav2Vec2Encoder(dim=g("encoder_embed_dim", 1024), layers=g("encoder_layers", 24),
                              heads=g("encoder_attention_heads", 16), ffn=g("encoder_ffn_embed_dim", 4096), dropout=0.0,
                              attn_dropout=0.0, layer_norm_first=g("layer_norm_first", True),
                              extractor_mode=g("extractor_mode", "layer_norm"), conv_bias=g("conv_bias", True),
                              pos_kernel=g("conv_pos", 128), pos_groups=g("conv_pos_groups", 16), **kw)
        load_wav2vec2_checkpoint(enc, state, verbose=False)
        weights = state.get("model", state)
        if "quantizer.vars" in weights:
            # pre-training checkpoints carry the product quantiser that labels the (unprojected) conv features
            from ..models.w2vbert import GumbelVectorQuantizer
            proj_w = weights["quantizer.weight_proj.weight"]
            groups = int(g("latent_groups", 2))
            entries = proj_w.shape[0] // groups
            vars_ = weights["quantizer.vars"].reshape(groups, entries, -1)
            q = GumbelVectorQuantizer(proj_w.shape[1], groups * vars_.shape[-1], groups, entries)
            with torch.no_grad():
                q.logits.weight.copy_(proj_w)
                q.logits.bias.copy_(weights["quantizer.weight_proj.bias"])
                q.codebook.copy_(vars_)
            enc.quantizer = q
    enc.eval()
    enc.to(device)
    quant = None
    for m in enc.modules():
        if m.__class__.__name__ == "GumbelVectorQuantizer":
            quant = m
    return enc, quant


def _batches(items: Iterable[Tuple[str, torch.Tensor]], max_samples: int):
    """Groups utterances so that (longest utterance x count) stays under ``max_samples``."""
    utts, waves, longest = [], [], 0
    for utt, w in items:
        new_longest = max(longest, w.numel())
        if waves and new_longest * (len(waves) + 1) > max_samples:
            yield utts, waves
            utts, waves, new_longest = [], [], w.numel()
        utts.append(utt)
        waves.append(w)
        longest = new_longest
    if waves:
        yield utts, waves


@torch.no_grad()
def encoder_frames(enc, waves: Sequence[torch.Tensor], layer: Optional[int] = None, device="cpu") -> List[torch.Tensor]:
    """Per utterance ``[frames, dim]``: the convolutional front end's output (``layer is None``) or the states after
    ``layer`` Transformer layers (0 = projected input of the first layer, -1 = all layers)."""
    lengths = torch.tensor([w.numel() for w in waves])
    wav = torch.zeros(len(waves), int(lengths.max()))
    for i, w in enumerate(waves):
        wav[i, :w.numel()] = w
    wav = wav.to(device)
    if layer is None:
        x = enc.extractor(wav)                                                    # [B, T, C]
        out_len = enc.extractor.output_lengths(lengths).clamp(max=x.shape[1])
        return [x[i, :int(out_len[i])].float().cpu() for i in range(len(waves))]
    from ..data.dataset import collate
    batch = collate([w.reshape(-1, 1) for w in waves], None, src_type="audio", round_to=1)
    src = batch.get("source")
    kept = enc.layers
    if layer >= 0:
        enc.layers = torch.nn.ModuleList(list(kept)[:layer])
    try:
        packed, seqs = enc(src.to(device) if torch.is_tensor(src) else src)
    finally:
        enc.layers = kept
    cu = seqs.cu.tolist()
    return [packed[cu[i]:cu[i + 1]].float().cpu() for i in range(len(waves))]


def extract_tdnn(model_path: str, wav_list: str, ark_path: str, scp_path: str, batch_samples: int = 16000 * 60,
                 layer: Optional[int] = None, device="cpu") -> int:
    """Writes one matrix per utterance into ``ark_path`` and its ``<utt> <ark>:<offset>`` line into ``scp_path``; returns
    the number of utterances."""
    enc, _ = load_speech_encoder(model_path, device)
    n = 0
    with open(ark_path, "wb") as ark, open(scp_path, "w") as scp:
        for utts, waves in _batches(read_wav_list(wav_list), batch_samples):
            for utt, f in zip(utts, encoder_frames(enc, waves, layer, device)):
                off = write_ark_matrix(ark, utt, f.numpy())
                scp.write("%s %s:%d\n" % (utt, os.path.abspath(ark_path), off))
                n += 1
    return n


def verify_tdnn(model_path: str, wav_list: str, scp_path: str, batch_samples: int = 16000 * 60, layer: Optional[int] = None,
                device="cpu", atol: float = 1e-5, rtol: float = 1e-5) -> Tuple[int, float]:
    """Recomputes the features of every recording of ``wav_list`` and compares them with the matrices ``scp_path`` points
    to (written earlier by ``extract_tdnn``): a check that a dump is still what the checkpoint produces, e.g. after the
    model or the audio pipeline changed.  Returns (utterances checked, largest absolute difference); raises
    ``AssertionError`` naming the first utterance outside the tolerance.  (reference: verify_wav2vec2_feat.py:91-114)"""
    enc, _ = load_speech_encoder(model_path, device)
    stored = read_scp(scp_path)
    n, worst = 0, 0.0
    for utts, waves in _batches(read_wav_list(wav_list), batch_samples):
        for utt, f in zip(utts, encoder_frames(enc, waves, layer, device)):
            if utt not in stored:
                raise AssertionError("utterance %s is not in %s" % (utt, scp_path))
            ref = torch.from_numpy(np.asarray(read_ark_matrix(*stored[utt]), dtype=np.float32))
            if ref.shape != f.shape:
                raise AssertionError("utterance %s: stored %s, recomputed %s" % (utt, tuple(ref.shape), tuple(f.shape)))
            diff = (ref - f).abs()
            worst = max(worst, float(diff.max()) if diff.numel() else 0.0)
            if not bool((diff <= atol + rtol * ref.abs()).all()):
                raise AssertionError("utterance %s differs from the stored features (max |diff| %.3g)" % (utt, float(diff.max())))
            n += 1
    return n, worst


@torch.no_grad()
def frame_codes(enc, quant, waves: Sequence[torch.Tensor], kmeans=None, layer: Optional[int] = None, device="cpu") -> List[List[str]]:
    """Per utterance one symbol per frame: ``"g0:g1"`` code indices of the product quantiser, or the k-means cluster."""
    feats = encoder_frames(enc, waves, layer, device)
    out = []
    for f in feats:
        if kmeans is not None:
            out.append([str(u) for u in kmeans.assign(f.to(kmeans.centroids.device)).tolist()])
            continue
        if quant is None:
            raise RuntimeError("the encoder has no quantiser: give a k-means model (-kmeans) instead")
        x = f.to(device)
        idx = quant.logits(x.float()).view(x.shape[0], quant.groups, quant.entries).argmax(-1).cpu()      # [T, groups]
        out.append([":".join(str(int(v)) for v in row) for row in idx])
    return out


def extract_codes(model_path: str, wav_list: str, out_path: str, batch_samples: int = 16000 * 60, kmeans_path: str = "",
                  layer: Optional[int] = None, device="cpu") -> int:
    enc, quant = load_speech_encoder(model_path, device)
    km = None
    if kmeans_path:
        from .kmeans import KMeans
        km = KMeans.load(torch.load(kmeans_path, map_location="cpu", weights_only=False))
    n = 0
    with open(out_path, "w") as fh:
        for utts, waves in _batches(read_wav_list(wav_list), batch_samples):
            for utt, codes in zip(utts, frame_codes(enc, quant, waves, km, layer, device)):
                fh.write("%s %s\n" % (utt, " ".join(codes)))
                n += 1
    return n


def main(argv=None, mode: str = "tdnn"):
    import argparse
    ap = argparse.ArgumentParser(description="wav2vec 2.0 feature extraction (%s)" % mode)
    ap.add_argument("-model", required=True, help="checkpoint of this framework or a fairseq wav2vec 2.0 checkpoint")
    ap.add_argument("-src", required=True, help="list of recordings: <utt> <wav> [<start> <end>]")
    ap.add_argument("-scp_output", default="output.scp")
    ap.add_argument("-scp", default="output.scp", help="verify mode: the scp file of the stored features")
    ap.add_argument("-ark_output", default="output.ark")
    ap.add_argument("-output", default="output.codes", help="codebook mode: text file with one utterance per line")
    ap.add_argument("-kmeans", default="", help="codebook mode: k-means model to label the frames with")
    ap.add_argument("-layer", type=int, default=None, help="states after this many Transformer layers instead of the conv front end")
    ap.add_argument("-batch_size", type=int, default=60, help="seconds of audio (longest x count) per batch")
    ap.add_argument("-gpu", type=int, default=-1)
    ap.add_argument("-fp16", action="store_true", help="accepted for command-line compatibility; extraction runs in fp32 / bf16")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", a.gpu) if a.gpu >= 0 and torch.cuda.is_available() else torch.device("cpu")
    if mode == "verify":
        n, worst = verify_tdnn(a.model, a.src, a.scp, a.batch_size * 16000, a.layer, dev)
        print("%d utterances match the stored features (largest difference %.3g)" % (n, worst))
        return n
    if mode == "tdnn":
        n = extract_tdnn(a.model, a.src, a.ark_output, a.scp_output, a.batch_size * 16000, a.layer, dev)
    else:
        n = extract_codes(a.model, a.src, a.output, a.batch_size * 16000, a.kmeans, a.layer, dev)
    print("%d utterances written" % n)
    return n
