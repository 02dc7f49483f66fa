"""Checkpoint I/O in the reference's on-disk layout.

A checkpoint is ``torch.save({'model', 'dicts', 'opt', 'epoch', 'itr', 'optim', 'scaler'})`` written to
``<save_model>_<metric>_<value:.6f>_e<epoch:.2f>.pt`` with retention of the best ``keep_save_files`` files
(reference: onmt/train_utils/mp_trainer.py:512-560, onmt/utils.py:52-79).  The ``model`` entry uses the
REFERENCE's parameter names, so files are interchangeable in both directions: this framework keeps fused
projections (``qkv``, ``kv``) internally and converts on save / load:

    encoder.layers.i.attn.qkv.weight  <->  cat(encoder.layer_modules.i.multihead.fc_{query,key,value}.function.linear.weight)
    decoder.layers.i.cross_attn.kv    <->  cat(...multihead_src.fc_{key,value}...)

Loading is tolerant in the same way as ``NMTModel.load_state_dict`` (onmt/modules/base_seq2seq.py:84-138):
positional buffers and the causal-mask buffer are ignored, keys missing from the file keep their fresh
initialisation, unknown keys are reported and skipped.
"""
from __future__ import annotations

import glob
import os
import re
from collections import OrderedDict
from typing import Dict, Optional

import torch

_SKIP_ON_LOAD = ("positional_encoder", "time_transformer", "decoder.mask")


def _ln(ref_prefix):
    return ref_prefix + ".layer_norm.function"


def transformer_to_reference(sd: Dict[str, torch.Tensor]) -> "OrderedDict[str, torch.Tensor]":
    """State dict of ``models.transformer.Transformer`` -> reference key names.  Parameters the reference layout has no
    name for here (residual gates of ``-rezero``, added convolution blocks, adapters ...) keep their own names, so that
    nothing a structure switch added is lost between saving and loading."""
    out = OrderedDict()
    native = sd

    class _Tracked(dict):
        def __init__(self, d):
            super().__init__(d)
            self.used = set()

        def __getitem__(self, k):
            self.used.add(k)
            return super().__getitem__(k)

    sd = _Tracked(native)

    def put(k, v):
        out[k] = v.detach().clone().float().cpu()

    def attn(prefix_new, prefix_ref, fused_qkv):
        H = sd[prefix_new + ".out.weight"].shape[0]
        if fused_qkv:
            w = sd[prefix_new + ".qkv.weight"]
            for j, n in enumerate(("query", "key", "value")):
                put("%s.fc_%s.function.linear.weight" % (prefix_ref, n), w[j * H:(j + 1) * H])
                if prefix_new + ".qkv.bias" in sd:
                    put("%s.fc_%s.function.linear.bias" % (prefix_ref, n), sd[prefix_new + ".qkv.bias"][j * H:(j + 1) * H])
        else:
            put("%s.fc_query.function.linear.weight" % prefix_ref, sd[prefix_new + ".q.weight"])
            kv = sd[prefix_new + ".kv.weight"]
            put("%s.fc_key.function.linear.weight" % prefix_ref, kv[:H])
            put("%s.fc_value.function.linear.weight" % prefix_ref, kv[H:])
            if prefix_new + ".q.bias" in sd:
                put("%s.fc_query.function.linear.bias" % prefix_ref, sd[prefix_new + ".q.bias"])
                put("%s.fc_key.function.linear.bias" % prefix_ref, sd[prefix_new + ".kv.bias"][:H])
                put("%s.fc_value.function.linear.bias" % prefix_ref, sd[prefix_new + ".kv.bias"][H:])
        put("%s.fc_concat.function.linear.weight" % prefix_ref, sd[prefix_new + ".out.weight"])
        if prefix_new + ".out.bias" in sd:
            put("%s.fc_concat.function.linear.bias" % prefix_ref, sd[prefix_new + ".out.bias"])

    def norm(new, ref):
        put(_ln(ref) + ".weight", sd[new + ".weight"])
        put(_ln(ref) + ".bias", sd[new + ".bias"])

    def ffn(new, ref):
        for a, b in (("fc1", "fc_1"), ("fc2", "fc_2")):
            put("%s.function.%s.linear.weight" % (ref, b), sd["%s.%s.weight" % (new, a)])
            put("%s.function.%s.linear.bias" % (ref, b), sd["%s.%s.bias" % (new, a)])

    put("encoder.word_lut.weight", sd["encoder.embed.weight"])
    n_enc = 1 + max([int(m.group(1)) for k in sd for m in [re.match(r"encoder\.layers\.(\d+)\.", k)] if m] + [-1])
    for i in range(n_enc):
        n, r = "encoder.layers.%d" % i, "encoder.layer_modules.%d" % i
        norm(n + ".attn_norm", r + ".preprocess_attn")
        attn(n + ".attn", r + ".multihead", True)
        if n + ".ffn_norm.weight" in sd:
            norm(n + ".ffn_norm", r + ".preprocess_ffn")
        if n + ".ffn.fc1.bias" in sd and n + ".ffn.fc2.bias" in sd:
            ffn(n + ".ffn", r + ".feedforward")
        if n + ".mcr_norm.weight" in sd:
            norm(n + ".mcr_norm", r + ".preprocess_mcr_ffn")
            ffn(n + ".mcr_ffn", r + ".mcr_feedforward")
    norm("encoder.final_norm", "encoder.postprocess_layer")
    put("decoder.word_lut.weight", sd["decoder.embed.weight"])
    n_dec = 1 + max([int(m.group(1)) for k in sd for m in [re.match(r"decoder\.layers\.(\d+)\.", k)] if m] + [-1])
    for i in range(n_dec):
        n, r = "decoder.layers.%d" % i, "decoder.layer_modules.%d" % i
        norm(n + ".self_norm", r + ".preprocess_attn")
        attn(n + ".self_attn", r + ".multihead_tgt", True)
        if n + ".cross_norm.weight" in sd:
            norm(n + ".cross_norm", r + ".preprocess_src_attn")
            attn(n + ".cross_attn", r + ".multihead_src", False)
        norm(n + ".ffn_norm", r + ".preprocess_ffn")
        if n + ".ffn.fc1.bias" in sd and n + ".ffn.fc2.bias" in sd:
            ffn(n + ".ffn", r + ".feedforward")
        if n + ".mcr_norm.weight" in sd:
            norm(n + ".mcr_norm", r + ".preprocess_mcr_ffn")
            ffn(n + ".mcr_ffn", r + ".mcr_feedforward")
    norm("decoder.final_norm", "decoder.postprocess_layer")
    put("generator.0.linear.weight", sd["generator.weight"])
    if "generator.bias" in sd:
        put("generator.0.linear.bias", sd["generator.bias"])
    for k, v in native.items():
        if k not in sd.used:
            put(k, v)
    return out


def transformer_from_reference(ref_sd: Dict[str, torch.Tensor], target_keys) -> "OrderedDict[str, torch.Tensor]":
    """Reference key names -> state dict of ``models.transformer.Transformer`` (only keys in ``target_keys``)."""
    out = OrderedDict()
    target_keys = set(target_keys)

    def get(k):
        return ref_sd.get(k)

    def set_if(k, v):
        if k in target_keys and v is not None:
            out[k] = v

    def cat(keys):
        parts = [get(k) for k in keys]
        return None if any(p is None for p in parts) else torch.cat(parts, 0)

    def attn(new, ref, fused_qkv):
        lin = lambda n, what: "%s.fc_%s.function.linear.%s" % (ref, n, what)
        if fused_qkv:
            set_if(new + ".qkv.weight", cat([lin(n, "weight") for n in ("query", "key", "value")]))
            set_if(new + ".qkv.bias", cat([lin(n, "bias") for n in ("query", "key", "value")]))
        else:
            set_if(new + ".q.weight", get(lin("query", "weight")))
            set_if(new + ".q.bias", get(lin("query", "bias")))
            set_if(new + ".kv.weight", cat([lin("key", "weight"), lin("value", "weight")]))
            set_if(new + ".kv.bias", cat([lin("key", "bias"), lin("value", "bias")]))
        set_if(new + ".out.weight", get(lin("concat", "weight")))
        set_if(new + ".out.bias", get(lin("concat", "bias")))

    def norm(new, ref):
        set_if(new + ".weight", get(_ln(ref) + ".weight"))
        set_if(new + ".bias", get(_ln(ref) + ".bias"))

    def ffn(new, ref):
        for a, b in (("fc1", "fc_1"), ("fc2", "fc_2")):
            set_if("%s.%s.weight" % (new, a), get("%s.function.%s.linear.weight" % (ref, b)))
            set_if("%s.%s.bias" % (new, a), get("%s.function.%s.linear.bias" % (ref, b)))

    set_if("encoder.embed.weight", get("encoder.word_lut.weight"))
    set_if("decoder.embed.weight", get("decoder.word_lut.weight"))
    layer_ids = lambda side: sorted({int(m.group(1)) for k in ref_sd for m in [re.match(side + r"\.layer_modules\.(\d+)\.", k)] if m})
    for i in layer_ids("encoder"):
        n, r = "encoder.layers.%d" % i, "encoder.layer_modules.%d" % i
        norm(n + ".attn_norm", r + ".preprocess_attn")
        attn(n + ".attn", r + ".multihead", True)
        norm(n + ".ffn_norm", r + ".preprocess_ffn")
        ffn(n + ".ffn", r + ".feedforward")
        norm(n + ".mcr_norm", r + ".preprocess_mcr_ffn")
        ffn(n + ".mcr_ffn", r + ".mcr_feedforward")
    norm("encoder.final_norm", "encoder.postprocess_layer")
    for i in layer_ids("decoder"):
        n, r = "decoder.layers.%d" % i, "decoder.layer_modules.%d" % i
        norm(n + ".self_norm", r + ".preprocess_attn")
        attn(n + ".self_attn", r + ".multihead_tgt", True)
        norm(n + ".cross_norm", r + ".preprocess_src_attn")
        attn(n + ".cross_attn", r + ".multihead_src", False)
        norm(n + ".ffn_norm", r + ".preprocess_ffn")
        ffn(n + ".ffn", r + ".feedforward")
        norm(n + ".mcr_norm", r + ".preprocess_mcr_ffn")
        ffn(n + ".mcr_ffn", r + ".mcr_feedforward")
    norm("decoder.final_norm", "decoder.postprocess_layer")
    set_if("generator.weight", get("generator.0.linear.weight"))
    set_if("generator.bias", get("generator.0.linear.bias"))
    for k, v in ref_sd.items():          # parameters saved under their own names (no reference name exists for them)
        if k in target_keys and k not in out:
            out[k] = v
    return out


def model_state_for_saving(model) -> Dict[str, torch.Tensor]:
    sd = {k: v for k, v in model.state_dict().items()}
    conv = getattr(model, "to_reference_state_dict", None)
    if conv is not None:
        return conv(sd)
    from ..models.transformer import Transformer
    if isinstance(model, Transformer):
        return transformer_to_reference(sd)
    return OrderedDict((k, v.detach().float().cpu()) for k, v in sd.items())


def load_model_state(model, state: Dict[str, torch.Tensor], strict: bool = False, verbose: bool = False):
    """Load a (reference- or native-named) state dict; returns (missing, unexpected) key lists."""
    own = model.state_dict()
    native_hits = sum(1 for k in state if k in own)
    conv = getattr(model, "from_reference_state_dict", None)
    from ..models.transformer import Transformer
    if native_hits < len(own) // 2:
        if conv is not None:
            state = conv(state, own.keys())
        elif isinstance(model, Transformer):
            state = transformer_from_reference(state, own.keys())
    filtered = {k: v for k, v in state.items() if k in own and not any(s in k for s in _SKIP_ON_LOAD)}
    unexpected = [k for k in state if k not in own and not any(s in k for s in _SKIP_ON_LOAD)]
    missing = [k for k in own if k not in filtered]
    if strict and (missing or unexpected):
        raise RuntimeError("state dict mismatch: missing %s, unexpected %s" % (missing[:5], unexpected[:5]))
    with torch.no_grad():
        for k, v in filtered.items():
            tgt = own[k]
            if tgt.shape != v.shape:
                if tgt.dim() == v.dim() and all(a >= b for a, b in zip(tgt.shape, v.shape)):
                    tgt[tuple(slice(0, s) for s in v.shape)].copy_(v)   # grown vocabulary / positions
                    continue
                raise RuntimeError("shape mismatch for %s: %s vs %s" % (k, tuple(tgt.shape), tuple(v.shape)))
            tgt.copy_(v)
    if verbose and (missing or unexpected):
        print("[checkpoint] missing keys: %d, unexpected keys: %d" % (len(missing), len(unexpected)))
    return missing, unexpected


def checkpoint_name(save_model: str, metric_name: str, value: float, epoch: float) -> str:
    return "%s_%s_%.6f_e%.2f.pt" % (save_model, metric_name, value, epoch)


def rng_state() -> dict:
    """Every random stream a training run draws from: Python, NumPy, torch (CPU and the current CUDA device) and the
    counter-based dropout seed of the fused kernels.  Saved with checkpoints so that a resumed run continues the same
    sequence of masks and shuffles (reference: whisper/trainers/trainer_pt_utils.py, RNG-state restore on resume)."""
    import random
    import numpy as np
    from .. import ops
    state = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state(),
             "dropout": (ops._Rng.seed, ops._Rng.counter)}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state()
        if ops.extension_available():
            # the device-resident word that every training step advances (added to the dropout seed inside the kernels)
            state["dropout_device_word"] = int(ops.ext().get_seed_tensor(torch.cuda.current_device()).item())
    return state


def restore_rng_state(state: Optional[dict]) -> bool:
    if not state:
        return False
    import random
    import numpy as np
    from .. import ops
    random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    torch.set_rng_state(state["torch"])
    if "cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda"])
    ops._Rng.seed, ops._Rng.counter = state["dropout"]
    if "dropout_device_word" in state and torch.cuda.is_available() and ops.extension_available():
        ops.ext().get_seed_tensor(torch.cuda.current_device()).fill_(int(state["dropout_device_word"]))
    return True


def save_checkpoint(path: str, model, dicts, opt, epoch: float, optim=None, itr=None, scaler=None, extra: Optional[dict] = None):
    ckpt = {"model": model_state_for_saving(model), "dicts": dicts, "opt": opt, "epoch": epoch, "itr": itr,
            "optim": optim.state_dict() if optim is not None else None, "scaler": scaler, "rng": rng_state()}
    if extra:
        ckpt.update(extra)
    tmp = path + ".tmp"
    torch.save(ckpt, tmp)
    os.replace(tmp, path)        # atomic: a crash never leaves a truncated file under the final name
    return path


def load_checkpoint(path: str):
    return torch.load(path, map_location="cpu", weights_only=False)


def prune_checkpoints(save_model: str, keep: int, metric_name: str = "ppl", lower_is_better: bool = True):
    """Keep the ``keep`` best files ``<save_model>_<metric>_<value>_e<epoch>.pt``, delete the rest."""
    files = glob.glob(glob.escape(save_model) + "_" + metric_name + "_*_e*.pt")
    scored = []
    for f in files:
        m = re.search(r"_%s_([-0-9.eE+naninf]+)_e([0-9.]+)\.pt$" % re.escape(metric_name), f)
        if m:
            try:
                scored.append((float(m.group(1)), f))
            except ValueError:
                continue
    scored.sort(key=lambda t: t[0], reverse=not lower_is_better)
    for _, f in scored[max(keep, 0):]:
        try:
            os.remove(f)
        except OSError:
            pass
    return [f for _, f in scored[:keep]]
