"""Loading pretrained weights, and state dicts in the reference's naming, for the pretrained-style families.

Three naming schemes meet here:

* **Hugging Face / fairseq module names** - what the files given with ``-enc_state_dict`` / ``-dec_state_dict`` /
  ``-wav2vec2_pretrained_model`` contain: ``layers.3.self_attn.q_proj.weight``, ``encoder_attn.k_proj.bias``,
  ``fc1.weight``, ``layernorm_embedding.weight`` ... (reference: onmt/model_factory.py:164-176, 333-350;
  onmt/models/speech_recognizer/wav2vec2.py:174-180 reads ``state['cfg']['model']`` and ``state['model']``).
* **the reference's "fast" layout** - what the reference's own checkpoints contain after ``optimize_model`` has
  merged the projections: ``self_attn.proj_weight`` holds q, k and v interleaved PER HEAD (``[heads, 3, d_head,
  d_model]`` flattened), ``encoder_attn.proj_weight_kv`` holds k and v as ``[heads, 2, d_head, d_model]``
  (pretrain_module/modeling_mbart.py:219-259, 475-513; fairseq_wav2vec2/fairseq_modules.py:458-497).
* **this framework's names** - fused ``qkv`` / ``kv`` projections stored as ``[q rows | k rows | v rows]``.

``to_native`` accepts either of the first two schemes per attention block, so one loader serves pretrained files
and reference checkpoints; ``to_reference`` writes the fast layout, which is what ``train/checkpoint.py`` saves for
these families so that the files stay interchangeable with the reference.
"""
from __future__ import annotations

import re
from collections import OrderedDict
from typing import Dict, Iterable, Optional

import torch


# ---------------------------------------------------------------------------------------------------------------
# fused-projection layouts
# ---------------------------------------------------------------------------------------------------------------
def deinterleave(w: torch.Tensor, heads: int, parts: int) -> torch.Tensor:
    """``[heads, parts, d_head, ...]`` (the reference's fast layout) -> ``[parts, heads, d_head, ...]``, i.e. the rows
    of q, then k, then v."""
    rest = tuple(w.shape[1:])
    d_head = w.shape[0] // (heads * parts)
    return w.reshape(heads, parts, d_head, *rest).transpose(0, 1).reshape(w.shape[0], *rest).contiguous()


def interleave(w: torch.Tensor, heads: int, parts: int) -> torch.Tensor:
    """Inverse of ``deinterleave``."""
    rest = tuple(w.shape[1:])
    d_head = w.shape[0] // (heads * parts)
    return w.reshape(parts, heads, d_head, *rest).transpose(0, 1).reshape(w.shape[0], *rest).contiguous()


def _zeros_like_bias(w: torch.Tensor) -> torch.Tensor:
    return torch.zeros(w.shape[0], dtype=w.dtype)


def _self_attn_to_native(src: Dict[str, torch.Tensor], sp: str, out: Dict[str, torch.Tensor], dp: str, heads: int):
    """Self-attention block ``sp`` (either naming) -> ``dp.qkv`` / ``dp.out``."""
    if sp + ".proj_weight" in src:                                   # reference fast layout
        out[dp + ".qkv.weight"] = deinterleave(src[sp + ".proj_weight"], heads, 3)
        if sp + ".proj_bias" in src:
            out[dp + ".qkv.bias"] = deinterleave(src[sp + ".proj_bias"], heads, 3)
    elif sp + ".in_proj_weight" in src:                              # already [q | k | v]
        out[dp + ".qkv.weight"] = src[sp + ".in_proj_weight"]
        if sp + ".in_proj_bias" in src:
            out[dp + ".qkv.bias"] = src[sp + ".in_proj_bias"]
    elif sp + ".q_proj.weight" in src:
        ws = [src[sp + ".%s_proj.weight" % n] for n in "qkv"]
        out[dp + ".qkv.weight"] = torch.cat(ws, 0)
        bs = [src.get(sp + ".%s_proj.bias" % n) for n in "qkv"]
        if any(b is not None for b in bs):                           # Whisper: the key projection has no bias
            out[dp + ".qkv.bias"] = torch.cat([b if b is not None else _zeros_like_bias(w) for b, w in zip(bs, ws)], 0)
    else:
        return
    for a, b in ((".out_proj.weight", ".out.weight"), (".out_proj.bias", ".out.bias")):
        if sp + a in src:
            out[dp + b] = src[sp + a]


def _cross_attn_to_native(src, sp, out, dp, heads):
    if sp + ".proj_weight_kv" in src:
        out[dp + ".kv.weight"] = deinterleave(src[sp + ".proj_weight_kv"], heads, 2)
        if sp + ".proj_bias_kv" in src:
            out[dp + ".kv.bias"] = deinterleave(src[sp + ".proj_bias_kv"], heads, 2)
        for cand in (".proj_weight_q", ".q_proj.weight"):
            if sp + cand in src:
                out[dp + ".q.weight"] = src[sp + cand]
        for cand in (".proj_bias_q", ".q_proj.bias"):
            if sp + cand in src:
                out[dp + ".q.bias"] = src[sp + cand]
    elif sp + ".k_proj.weight" in src:
        wk, wv = src[sp + ".k_proj.weight"], src[sp + ".v_proj.weight"]
        out[dp + ".kv.weight"] = torch.cat([wk, wv], 0)
        bk, bv = src.get(sp + ".k_proj.bias"), src.get(sp + ".v_proj.bias")
        if bk is not None or bv is not None:
            out[dp + ".kv.bias"] = torch.cat([bk if bk is not None else _zeros_like_bias(wk),
                                              bv if bv is not None else _zeros_like_bias(wv)], 0)
        out[dp + ".q.weight"] = src[sp + ".q_proj.weight"]
        if sp + ".q_proj.bias" in src:
            out[dp + ".q.bias"] = src[sp + ".q_proj.bias"]
    else:
        return
    for a, b in ((".out_proj.weight", ".out.weight"), (".out_proj.bias", ".out.bias")):
        if sp + a in src:
            out[dp + b] = src[sp + a]


# ---------------------------------------------------------------------------------------------------------------
# whole stacks: Hugging Face / fairseq module names -> this framework's names
# ---------------------------------------------------------------------------------------------------------------
_NORM = ((".weight", ".weight"), (".bias", ".bias"))


def _copy(src, sk, out, dk):
    if sk in src:
        out[dk] = src[sk]


def _strip_prefix(sd: Dict[str, torch.Tensor], candidates: Iterable[str]) -> Dict[str, torch.Tensor]:
    """Drop the first of ``candidates`` that prefixes at least one key ("model.decoder.", "decoder.", ...)."""
    for pre in candidates:
        hit = {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}
        if hit:
            return hit
    return dict(sd)


def _layer_ids(sd, prefix="layers."):
    ids = set()
    for k in sd:
        m = re.match(re.escape(prefix) + r"(\d+)\.", k)
        if m:
            ids.add(int(m.group(1)))
    return sorted(ids)


def decoder_to_native(sd: Dict[str, torch.Tensor], heads: int, interleaved_ffn: bool = False) -> "OrderedDict[str, torch.Tensor]":
    """mBART / BART / M2M-100 / Whisper / DeltaLM decoder (module-level names, either attention layout) ->
    ``PretrainedStyleDecoder`` names.  DeltaLM's extra feed-forward block between the two attentions is ``fc3`` /
    ``fc4`` + ``ffn_layer_norm`` there and ``mid_ffn`` / ``mid_norm`` here."""
    sd = _strip_prefix(sd, ("model.decoder.", "decoder."))
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    _copy(sd, "embed_tokens.weight", out, "embed.weight")
    _copy(sd, "embed_positions.weight", out, "embed.pos")
    for a, b in _NORM:
        _copy(sd, "layernorm_embedding" + a, out, "emb_norm" + b)
        _copy(sd, "layer_norm" + a, out, "final_norm" + b)
    for i in _layer_ids(sd):
        s, d = "layers.%d" % i, "layers.%d" % i
        _self_attn_to_native(sd, s + ".self_attn", out, d + ".self_attn", heads)
        _cross_attn_to_native(sd, s + ".encoder_attn", out, d + ".cross_attn", heads)
        for a, b in _NORM:
            _copy(sd, s + ".self_attn_layer_norm" + a, out, d + ".self_norm" + b)
            _copy(sd, s + ".encoder_attn_layer_norm" + a, out, d + ".cross_norm" + b)
            _copy(sd, s + ".final_layer_norm" + a, out, d + ".ffn_norm" + b)
            _copy(sd, s + ".fc1" + a, out, d + ".ffn.fc1" + b)
            _copy(sd, s + ".fc2" + a, out, d + ".ffn.fc2" + b)
            if interleaved_ffn:
                _copy(sd, s + ".fc3" + a, out, d + ".mid_ffn.fc1" + b)
                _copy(sd, s + ".fc4" + a, out, d + ".mid_ffn.fc2" + b)
                _copy(sd, s + ".ffn_layer_norm" + a, out, d + ".mid_norm" + b)
    return out


def text_encoder_to_native(sd: Dict[str, torch.Tensor], heads: int) -> "OrderedDict[str, torch.Tensor]":
    """mBART / BART / M2M-100 / DeltaLM text encoder -> ``PretrainedStyleEncoder`` names."""
    sd = _strip_prefix(sd, ("model.encoder.", "encoder."))
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    _copy(sd, "embed_tokens.weight", out, "embed.weight")
    _copy(sd, "embed_positions.weight", out, "embed.pos")
    for a, b in _NORM:
        _copy(sd, "layernorm_embedding" + a, out, "emb_norm" + b)
        _copy(sd, "layer_norm" + a, out, "final_norm" + b)
    for i in _layer_ids(sd):
        s, d = "layers.%d" % i, "layers.%d" % i
        _self_attn_to_native(sd, s + ".self_attn", out, d + ".attn", heads)
        for a, b in _NORM:
            _copy(sd, s + ".self_attn_layer_norm" + a, out, d + ".attn_norm" + b)
            _copy(sd, s + ".final_layer_norm" + a, out, d + ".ffn_norm" + b)
            _copy(sd, s + ".fc1" + a, out, d + ".ffn.fc1" + b)
            _copy(sd, s + ".fc2" + a, out, d + ".ffn.fc2" + b)
    return out


def whisper_encoder_to_native(sd: Dict[str, torch.Tensor], heads: int) -> "OrderedDict[str, torch.Tensor]":
    """Whisper audio encoder (``conv1``, ``conv2``, pre-LN layers, ``layer_norm``) -> ``WhisperEncoder`` names.  The
    fixed sinusoidal ``embed_positions`` table of the file is not copied: this encoder computes the same table."""
    sd = _strip_prefix(sd, ("model.encoder.", "encoder."))
    out = text_encoder_to_native(sd, heads)
    out.pop("embed.pos", None)
    for name in ("conv1", "conv2"):
        for a, b in _NORM:
            _copy(sd, name + a, out, name + b)
    return out


def wav2vec2_to_native(sd: Dict[str, torch.Tensor], heads: int, extractor_mode: str = "layer_norm") -> "OrderedDict[str, torch.Tensor]":
    """fairseq wav2vec 2.0 / HuBERT model state (``state['model']``) -> ``Wav2Vec2Encoder`` names.

    ``feature_extractor.conv_layers.i.0`` is the convolution; its normalisation sits at ``.2.1`` in ``layer_norm``
    mode (Sequential(TransposeLast, LayerNorm, TransposeLast)) and at ``.2`` (GroupNorm, first layer only) otherwise.
    The positional convolution keeps its weight-norm parametrisation: ``weight_g`` / ``weight_v`` of the file are
    ``parametrizations.weight.original0`` / ``original1`` here.  Quantiser, ``final_proj`` and other pre-training heads
    are ignored, as in the reference (onmt/models/speech_recognizer/wav2vec2.py:196-230 removes them)."""
    sd = _strip_prefix(sd, ("w2v_encoder.w2v_model.", "wav2vec_encoder.", "w2v_model."))
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    _copy(sd, "mask_emb", out, "mask_emb")
    i = 0
    while "feature_extractor.conv_layers.%d.0.weight" % i in sd:
        p = "feature_extractor.conv_layers.%d" % i
        _copy(sd, p + ".0.weight", out, "extractor.convs.%d.weight" % i)
        _copy(sd, p + ".0.bias", out, "extractor.convs.%d.bias" % i)
        for a, b in _NORM:
            _copy(sd, p + ".2.1" + a, out, "extractor.norms.%d" % i + b)      # layer_norm mode
            _copy(sd, p + ".2" + a, out, "extractor.norms.%d" % i + b)        # group norm (default mode, layer 0)
        i += 1
    for a, b in _NORM:
        _copy(sd, "layer_norm" + a, out, "feat_norm" + b)
        _copy(sd, "post_extract_proj" + a, out, "post_extract_proj" + b)
        _copy(sd, "encoder.layer_norm" + a, out, "input_norm" + b)
    _copy(sd, "encoder.pos_conv.0.bias", out, "pos_conv.conv.bias")
    _copy(sd, "encoder.pos_conv.0.weight_g", out, "pos_conv.conv.parametrizations.weight.original0")
    _copy(sd, "encoder.pos_conv.0.weight_v", out, "pos_conv.conv.parametrizations.weight.original1")
    _copy(sd, "encoder.pos_conv.0.parametrizations.weight.original0", out, "pos_conv.conv.parametrizations.weight.original0")
    _copy(sd, "encoder.pos_conv.0.parametrizations.weight.original1", out, "pos_conv.conv.parametrizations.weight.original1")
    for i in _layer_ids(sd, "encoder.layers."):
        s, d = "encoder.layers.%d" % i, "layers.%d" % i
        _self_attn_to_native(sd, s + ".self_attn", out, d + ".attn", heads)
        for a, b in _NORM:
            _copy(sd, s + ".self_attn_layer_norm" + a, out, d + ".attn_norm" + b)
            _copy(sd, s + ".final_layer_norm" + a, out, d + ".ffn_norm" + b)
            _copy(sd, s + ".fc1" + a, out, d + ".ffn.fc1" + b)
            _copy(sd, s + ".fc2" + a, out, d + ".ffn.fc2" + b)
        # WavLM's gated relative position bias
        _copy(sd, s + ".self_attn.relative_attention_bias.weight", out, d + ".attn.relative_attention_bias.weight")
        _copy(sd, s + ".self_attn.grep_a", out, d + ".attn.grep_a")
        for a, b in _NORM:
            _copy(sd, s + ".self_attn.grep_linear" + a, out, d + ".attn.grep_linear" + b)
    return out


# ---------------------------------------------------------------------------------------------------------------
# this framework's names -> the reference's checkpoint names (fast layout)
# ---------------------------------------------------------------------------------------------------------------
def _self_attn_to_reference(src, sp, out, dp, heads):
    if sp + ".qkv.weight" not in src:
        return
    out[dp + ".proj_weight"] = interleave(src[sp + ".qkv.weight"], heads, 3)
    if sp + ".qkv.bias" in src:
        out[dp + ".proj_bias"] = interleave(src[sp + ".qkv.bias"], heads, 3)
    _copy(src, sp + ".out.weight", out, dp + ".out_proj.weight")
    _copy(src, sp + ".out.bias", out, dp + ".out_proj.bias")


def _cross_attn_to_reference(src, sp, out, dp, heads):
    if sp + ".kv.weight" not in src:
        return
    out[dp + ".proj_weight_kv"] = interleave(src[sp + ".kv.weight"], heads, 2)
    if sp + ".kv.bias" in src:
        out[dp + ".proj_bias_kv"] = interleave(src[sp + ".kv.bias"], heads, 2)
    _copy(src, sp + ".q.weight", out, dp + ".q_proj.weight")
    _copy(src, sp + ".q.bias", out, dp + ".q_proj.bias")
    _copy(src, sp + ".out.weight", out, dp + ".out_proj.weight")
    _copy(src, sp + ".out.bias", out, dp + ".out_proj.bias")


def decoder_to_reference(sd: Dict[str, torch.Tensor], heads: int, interleaved_ffn: bool = False) -> "OrderedDict[str, torch.Tensor]":
    """``PretrainedStyleDecoder`` state (keys relative to the decoder) -> the reference's decoder names, fast layout."""
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    _copy(sd, "embed.weight", out, "embed_tokens.weight")
    _copy(sd, "embed.pos", out, "embed_positions.weight")
    for a, b in _NORM:
        _copy(sd, "emb_norm" + a, out, "layernorm_embedding" + b)
        _copy(sd, "final_norm" + a, out, "layer_norm" + b)
    for i in _layer_ids(sd):
        s = d = "layers.%d" % i
        _self_attn_to_reference(sd, s + ".self_attn", out, d + ".self_attn", heads)
        _cross_attn_to_reference(sd, s + ".cross_attn", out, d + ".encoder_attn", heads)
        for a, b in _NORM:
            _copy(sd, s + ".self_norm" + a, out, d + ".self_attn_layer_norm" + b)
            _copy(sd, s + ".cross_norm" + a, out, d + ".encoder_attn_layer_norm" + b)
            _copy(sd, s + ".ffn_norm" + a, out, d + ".final_layer_norm" + b)
            _copy(sd, s + ".ffn.fc1" + a, out, d + ".fc1" + b)
            _copy(sd, s + ".ffn.fc2" + a, out, d + ".fc2" + b)
            if interleaved_ffn:
                _copy(sd, s + ".mid_ffn.fc1" + a, out, d + ".fc3" + b)
                _copy(sd, s + ".mid_ffn.fc2" + a, out, d + ".fc4" + b)
                _copy(sd, s + ".mid_norm" + a, out, d + ".ffn_layer_norm" + b)
    return out


def text_encoder_to_reference(sd: Dict[str, torch.Tensor], heads: int) -> "OrderedDict[str, torch.Tensor]":
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    _copy(sd, "embed.weight", out, "embed_tokens.weight")
    _copy(sd, "embed.pos", out, "embed_positions.weight")
    for a, b in _NORM:
        _copy(sd, "emb_norm" + a, out, "layernorm_embedding" + b)
        _copy(sd, "final_norm" + a, out, "layer_norm" + b)
        _copy(sd, "conv1" + a, out, "conv1" + b)
        _copy(sd, "conv2" + a, out, "conv2" + b)
    for i in _layer_ids(sd):
        s = d = "layers.%d" % i
        _self_attn_to_reference(sd, s + ".attn", out, d + ".self_attn", heads)
        for a, b in _NORM:
            _copy(sd, s + ".attn_norm" + a, out, d + ".self_attn_layer_norm" + b)
            _copy(sd, s + ".ffn_norm" + a, out, d + ".final_layer_norm" + b)
            _copy(sd, s + ".ffn.fc1" + a, out, d + ".fc1" + b)
            _copy(sd, s + ".ffn.fc2" + a, out, d + ".fc2" + b)
    return out


def wav2vec2_to_reference(sd: Dict[str, torch.Tensor], heads: int, layer_norm_mode: bool = True) -> "OrderedDict[str, torch.Tensor]":
    """``Wav2Vec2Encoder`` state -> fairseq names with the reference's fast attention layout."""
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    _copy(sd, "mask_emb", out, "mask_emb")
    i = 0
    while "extractor.convs.%d.weight" % i in sd:
        p = "feature_extractor.conv_layers.%d" % i
        _copy(sd, "extractor.convs.%d.weight" % i, out, p + ".0.weight")
        _copy(sd, "extractor.convs.%d.bias" % i, out, p + ".0.bias")
        for a, b in _NORM:
            _copy(sd, "extractor.norms.%d" % i + a, out, p + (".2.1" if layer_norm_mode else ".2") + b)
        i += 1
    for a, b in _NORM:
        _copy(sd, "feat_norm" + a, out, "layer_norm" + b)
        _copy(sd, "post_extract_proj" + a, out, "post_extract_proj" + b)
        _copy(sd, "input_norm" + a, out, "encoder.layer_norm" + b)
    _copy(sd, "pos_conv.conv.bias", out, "encoder.pos_conv.0.bias")
    _copy(sd, "pos_conv.conv.parametrizations.weight.original0", out, "encoder.pos_conv.0.weight_g")
    _copy(sd, "pos_conv.conv.parametrizations.weight.original1", out, "encoder.pos_conv.0.weight_v")
    for i in _layer_ids(sd):
        s, d = "layers.%d" % i, "encoder.layers.%d" % i
        _self_attn_to_reference(sd, s + ".attn", out, d + ".self_attn", heads)
        for a, b in _NORM:
            _copy(sd, s + ".attn_norm" + a, out, d + ".self_attn_layer_norm" + b)
            _copy(sd, s + ".ffn_norm" + a, out, d + ".final_layer_norm" + b)
            _copy(sd, s + ".ffn.fc1" + a, out, d + ".fc1" + b)
            _copy(sd, s + ".ffn.fc2" + a, out, d + ".fc2" + b)
    return out


# ---------------------------------------------------------------------------------------------------------------
# entry points
# ---------------------------------------------------------------------------------------------------------------
def _load_file(path: str):
    obj = torch.load(path, map_location="cpu", weights_only=False)
    return obj


def _heads_of(module) -> int:
    for m in module.modules():
        h = getattr(m, "heads", None)
        if isinstance(h, int) and h > 0:
            return h
    return 1


def _assign(module, native_sd: Dict[str, torch.Tensor], what: str, verbose: bool = True, strict_shapes: bool = False):
    """Copy ``native_sd`` into ``module``; vocabulary / position tables may be larger on either side (the common
    prefix of rows is copied).  Returns (loaded, missing, unexpected)."""
    own = module.state_dict()
    loaded, unexpected = 0, []
    with torch.no_grad():
        for k, v in native_sd.items():
            if k not in own:
                unexpected.append(k)
                continue
            tgt = own[k]
            if tgt.shape == v.shape:
                tgt.copy_(v)
            elif not strict_shapes and tgt.dim() == v.dim() and tgt.shape[1:] == v.shape[1:]:
                n = min(tgt.shape[0], v.shape[0])
                tgt[:n].copy_(v[:n])
            else:
                raise RuntimeError("%s: shape of %s is %s in the file and %s in the model" % (what, k, tuple(v.shape), tuple(tgt.shape)))
            loaded += 1
    missing = [k for k in own if k not in native_sd]
    if verbose:
        print("[INFO] %s: %d tensors loaded, %d of the model's not in the file, %d of the file's unused"
              % (what, loaded, len(missing), len(unexpected)))
    return loaded, missing, unexpected


def load_decoder_state(decoder, sd: Dict[str, torch.Tensor], verbose: bool = True):
    """``-dec_state_dict``: a decoder's state dict in module-level names (either attention layout)."""
    inter = any(getattr(l, "interleaved_ffn", False) for l in getattr(decoder, "layers", []))
    native = decoder_to_native(sd, _heads_of(decoder), interleaved_ffn=inter)
    if not native:
        raise RuntimeError("no decoder weights recognised in the file (first keys: %s)" % list(sd.keys())[:5])
    return _assign(decoder, native, "decoder weights", verbose)


def load_text_encoder_state(encoder, sd: Dict[str, torch.Tensor], verbose: bool = True):
    native = text_encoder_to_native(sd, _heads_of(encoder))
    if not native:
        raise RuntimeError("no encoder weights recognised in the file (first keys: %s)" % list(sd.keys())[:5])
    return _assign(encoder, native, "encoder weights", verbose)


def load_whisper_state(model, sd: Dict[str, torch.Tensor], verbose: bool = True):
    """A Whisper checkpoint (``model.encoder.*`` / ``model.decoder.*`` [+ ``proj_out``]) into a ``whisper`` model."""
    if any(k.startswith("model.") for k in sd):
        sd = {k[len("model."):]: v for k, v in sd.items() if k.startswith("model.")}
    enc = {k: v for k, v in sd.items() if k.startswith("encoder.")}
    dec = {k: v for k, v in sd.items() if k.startswith("decoder.")}
    out = []
    if enc:
        out.append(_assign(model.encoder, whisper_encoder_to_native(enc, _heads_of(model.encoder)), "Whisper encoder", verbose))
    if dec:
        out.append(load_decoder_state(model.decoder, dec, verbose))
    return out


def load_wav2vec2_checkpoint(encoder, path_or_state, verbose: bool = True):
    """``-wav2vec2_pretrained_model``: a fairseq checkpoint ``{'cfg': {'model': ...}, 'model': state_dict}`` (or a bare
    state dict).  Returns the ``cfg['model']`` mapping of the file (empty for a bare state dict)."""
    state = _load_file(path_or_state) if isinstance(path_or_state, str) else path_or_state
    cfg = {}
    if isinstance(state, dict) and "model" in state and isinstance(state["model"], dict):
        c = state.get("cfg") or state.get("args") or {}
        cfg = c.get("model", c) if isinstance(c, dict) else vars(c)
        state = state["model"]
    native = wav2vec2_to_native(state, _heads_of(encoder))
    if not native:
        raise RuntimeError("no wav2vec 2.0 weights recognised in the file (first keys: %s)" % list(state.keys())[:5])
    _assign(encoder, native, "wav2vec 2.0 encoder", verbose)
    return cfg


def wav2vec2_config_from_checkpoint(path: str) -> dict:
    """The architecture fields of a fairseq checkpoint (``state['cfg']['model']``), as the reference reads them
    (onmt/models/speech_recognizer/wav2vec2.py:174-180), without keeping the weights in memory afterwards."""
    state = _load_file(path)
    c = state.get("cfg") or state.get("args") or {}
    c = c.get("model", c) if isinstance(c, dict) else vars(c)
    return dict(c) if isinstance(c, dict) else dict(vars(c))


def copy_embeddings_by_token(dst_weight: torch.Tensor, dst_dict, src_weight: torch.Tensor, src_dict) -> int:
    """Rows of ``src_weight`` whose token also exists in ``dst_dict`` are copied to that token's row: how
    ``-load_encoder_from`` / ``-load_decoder_from`` carry embeddings across different vocabularies
    (reference: onmt/train_utils/mp_trainer.py:438-510).  Returns the number of rows copied."""
    n = 0
    labels = getattr(src_dict, "idxToLabel", None) or {}
    with torch.no_grad():
        for idx, word in labels.items():
            if idx >= src_weight.shape[0]:
                continue
            j = dst_dict.lookup(word)
            if j is not None and j < dst_weight.shape[0]:
                dst_weight[j].copy_(src_weight[idx])
                n += 1
    return n


def load_side_from_checkpoint(model, path: str, side: str, dicts=None, verbose: bool = True):
    """``-load_encoder_from`` / ``-load_decoder_from``: take one side of another trained model (a checkpoint of this
    framework or of the reference).  Shapes that differ only in the vocabulary dimension are matched by token when
    both dictionaries are known, else by row index."""
    from ..train.checkpoint import load_model_state
    ckpt = _load_file(path)
    state = ckpt["model"] if isinstance(ckpt, dict) and "model" in ckpt else ckpt
    # bring the whole file into this model's naming with the usual tolerant loader on a scratch copy of the names
    own = model.state_dict()
    conv = getattr(model, "from_reference_state_dict", None)
    native_hits = sum(1 for k in state if k in own)
    if native_hits < len(own) // 2:
        if conv is not None:
            state = conv(state, own.keys())
        else:
            from ..models.transformer import Transformer
            from ..train.checkpoint import transformer_from_reference
            if isinstance(model, Transformer):
                state = transformer_from_reference(state, own.keys())
    prefix = side + "."
    picked = {k: v for k, v in state.items() if k.startswith(prefix)}
    if side == "decoder":
        picked.update({k: v for k, v in state.items() if k.startswith("generator.")})
    if not picked:
        raise RuntimeError("%s holds no %s weights" % (path, side))
    src_dicts = ckpt.get("dicts") if isinstance(ckpt, dict) else None
    which = "src" if side == "encoder" else "tgt"
    loaded = 0
    with torch.no_grad():
        for k, v in picked.items():
            if k not in own:
                continue
            tgt = own[k]
            if tgt.shape == v.shape:
                tgt.copy_(v)
            elif tgt.dim() == 2 and v.dim() == 2 and tgt.shape[1] == v.shape[1] and ("embed.weight" in k or k.startswith("generator.")):
                if dicts is not None and src_dicts is not None and which in dicts and which in src_dicts:
                    copy_embeddings_by_token(tgt, dicts[which], v, src_dicts[which])
                else:
                    n = min(tgt.shape[0], v.shape[0])
                    tgt[:n].copy_(v[:n])
            elif tgt.dim() == 1 and v.dim() == 1 and k.startswith("generator."):
                n = min(tgt.shape[0], v.shape[0])
                tgt[:n].copy_(v[:n])
            else:
                continue
            loaded += 1
    if verbose:
        print("[INFO] %s weights taken from %s: %d tensors" % (side, path, loaded))
    return loaded


def load_pretrained_parts(model, opt, dicts=None, verbose: Optional[bool] = None):
    """Everything the command line names: ``-wav2vec2_pretrained_model`` (only when it is a file), ``-enc_state_dict``,
    ``-dec_state_dict``, ``-load_encoder_from``, ``-load_decoder_from``."""
    import os
    verbose = bool(getattr(opt, "verbose", False)) if verbose is None else verbose
    done = []
    enc, dec = getattr(model, "encoder", None), getattr(model, "decoder", None)
    w2v = getattr(opt, "wav2vec2_pretrained_model", "") or ""
    if w2v and os.path.isfile(w2v) and enc is not None and hasattr(enc, "extractor"):
        load_wav2vec2_checkpoint(enc, w2v, verbose)
        done.append("wav2vec2_pretrained_model")
    esd = getattr(opt, "enc_state_dict", "") or ""
    if esd and enc is not None:
        if not os.path.isfile(esd):
            raise FileNotFoundError("-enc_state_dict %s does not exist" % esd)
        sd = _load_file(esd)
        sd = sd.get("model", sd) if isinstance(sd, dict) and "model" in sd and isinstance(sd["model"], dict) else sd
        if hasattr(enc, "extractor"):
            load_wav2vec2_checkpoint(enc, sd, verbose)
        elif hasattr(enc, "conv1"):
            _assign(enc, whisper_encoder_to_native(sd, _heads_of(enc)), "Whisper encoder", verbose)
        else:
            load_text_encoder_state(enc, sd, verbose)
        done.append("enc_state_dict")
    dsd = getattr(opt, "dec_state_dict", "") or ""
    if dsd and dec is not None:
        if not os.path.isfile(dsd):
            raise FileNotFoundError("-dec_state_dict %s does not exist" % dsd)
        sd = _load_file(dsd)
        sd = sd.get("model", sd) if isinstance(sd, dict) and "model" in sd and isinstance(sd["model"], dict) else sd
        load_decoder_state(dec, sd, verbose)
        if getattr(model, "generator", None) is not None and hasattr(model, "tie_weights") and \
                model.generator.weight.shape == dec.embed.weight.shape:
            model.tie_weights()
        done.append("dec_state_dict")
    for flag, side in (("load_encoder_from", "encoder"), ("load_decoder_from", "decoder")):
        path = getattr(opt, flag, "") or ""
        if path:
            load_side_from_checkpoint(model, path, side, dicts, verbose)
            done.append(flag)
    return done
