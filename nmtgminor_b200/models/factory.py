"""Model factory: ``opt.model`` -> model object.

A registry maps the reference's model names (onmt/model_factory.py:102-731) to builder functions so that
families can be added without touching a central if-chain.  ``build_model`` is the single entry point used
by trainers and translators: it validates the options, builds the model, applies ``-init`` / ``-init_embedding``,
loads pretrained sub-modules (``-enc_state_dict``, ``-dec_state_dict``, ``-wav2vec2_pretrained_model``) and freezes
what the ``-freeze_*`` options name.  ``optimize_model`` exists for API parity (projections are born fused).
"""
from __future__ import annotations

from typing import Callable, Dict

_REGISTRY: Dict[str, Callable] = {}


def register(*names):
    def deco(fn):
        for n in names:
            _REGISTRY[n] = fn
        return fn
    return deco


def build_model(opt, dicts, remove_pretrain: bool = False, constants=None):
    _load_builders()
    from ..options import backward_compatible
    opt = backward_compatible(opt)
    name = getattr(opt, "model", "transformer")
    if getattr(opt, "model_type", "") == "lm" or name in ("TransformerXL", "transformer_xl_lm", "transformer_xl"):
        return _REGISTRY["transformer_xl_lm"](opt, dicts)
    if (getattr(opt, "activation_layer", "linear_relu_linear") or "linear_relu_linear") != "linear_relu_linear":
        raise NotImplementedError("-activation_layer %s changes the feed-forward blocks of the Transformer-XL language model "
                                  "only (as in the reference); model '%s' keeps -ffn_activation" % (opt.activation_layer, name))
    if name not in _REGISTRY:
        raise NotImplementedError("unknown model %r; registered: %s" % (name, sorted(_REGISTRY)))
    from ..options import validate_model_options
    validate_model_options(opt)
    if getattr(opt, "fusion", False):
        return build_fusion(opt, dicts, remove_pretrain)
    model = _REGISTRY[name](opt, dicts)
    init_model_parameters(model, opt)
    if getattr(opt, "no_decoder", False) and not getattr(model, "ctc_only", False):
        raise NotImplementedError("-no_decoder builds encoder-only CTC models of the wav2vec 2.0 family (wav2vec2_bert, "
                                  "wav2vec2_transformer); model '%s' keeps its decoder" % name)
    if int(getattr(opt, "predict_language", 0) or 0) > 0:
        if not hasattr(model, "enable_language_prediction"):
            raise NotImplementedError("-predict_language is built for the speech-to-text models")
        from .transformer import _n_languages
        model.enable_language_prediction(_n_languages(dicts))
    if int(getattr(opt, "batch_ensemble", 0) or 0) > 0:
        from ..modules.batch_ensemble import convert_to_batch_ensemble
        convert_to_batch_ensemble(model, int(opt.batch_ensemble))
    if getattr(opt, "rotary_position_encoding", False) and not any(getattr(m, "rotary", False) for m in model.modules()):
        raise NotImplementedError("-rotary_position_encoding is built for the wav2vec 2.0 family encoders; model '%s' has no "
                                  "rotary attention" % getattr(opt, "model", "?"))
    for flag, side in (("wav2vec_adapter", "encoder"), ("decoder_adapter", "decoder")):
        if int(getattr(opt, flag, 0) or 0) > 0 and getattr(getattr(model, side, None), "adapters", None) is None:
            raise NotImplementedError("-%s: the %s of model '%s' has no language-adapter slots (built for the wav2vec 2.0 "
                                      "family encoders and the pretrained-style decoders)" % (flag, side, getattr(opt, "model", "?")))
    if float(getattr(opt, "weight_drop", 0.0) or 0.0) > 0:
        from .layers import FeedForward
        for m in model.modules():
            if isinstance(m, FeedForward):
                m.weight_drop = float(opt.weight_drop)
    if getattr(opt, "no_ffn", False) or getattr(opt, "depthwise_conv", False):
        from .layers import EncoderLayer
        layers = [m for m in getattr(model, "encoder", model).modules() if isinstance(m, EncoderLayer)]
        if not layers:
            raise NotImplementedError("-no_ffn / -depthwise_conv change the standard encoder layers; the encoder of model "
                                      "'%s' is not built from them" % getattr(opt, "model", "?"))
        for m in layers:
            if getattr(opt, "depthwise_conv", False):
                m.add_depthwise_conv(int(getattr(opt, "conv_kernel", 31) or 31))
            if getattr(opt, "no_ffn", False):
                m.drop_ffn()
    if getattr(opt, "branchformer", False):
        from .layers import EncoderLayer
        layers = [m for m in getattr(model, "encoder", model).modules() if isinstance(m, EncoderLayer)]
        if not layers:
            raise NotImplementedError("-branchformer adds a cgMLP branch to the standard encoder layers; the encoder of "
                                      "model '%s' is not built from them" % getattr(opt, "model", "?"))
        for m in layers:
            m.add_branchformer(int(getattr(opt, "conv_kernel", 31) or 31))
    if getattr(opt, "favor_attention", False):
        from .layers import SelfAttention
        mods = [m for m in getattr(model, "encoder", model).modules() if isinstance(m, SelfAttention) and not m.causal]
        if not mods:
            raise NotImplementedError("-favor_attention replaces the encoder's self-attention; the encoder of model '%s' has "
                                      "none of the standard attention blocks" % getattr(opt, "model", "?"))
        for i, m in enumerate(mods):
            m.enable_favor(seed=int(getattr(opt, "seed", 0) or 0) + i)
    if getattr(opt, "stochastic_sublayer", False):
        from .layers import _LayerOptions
        for m in model.modules():
            if isinstance(m, _LayerOptions):
                m.stochastic_sublayer = True
    if not remove_pretrain:          # a full checkpoint is about to be loaded: its weights replace the pretrained ones
        load_pretrained_parts(model, opt, dicts)
    apply_freeze_options(model, opt)
    aux = dicts.get("aux_tgt") if hasattr(dicts, "get") else None
    if aux is not None and getattr(model, "ctc_linear", None) is not None:
        # "triangle" corpora: the CTC head predicts the auxiliary target (the transcript), which has its own vocabulary
        import torch.nn as nn
        model.ctc_linear = nn.Linear(model.ctc_linear.in_features, aux.size())
        model.ctc_on_aux = True
    return model


def build_fusion(opt, dicts, remove_pretrain: bool = False):
    """``-fusion -lm_checkpoint lm.pt``: the translation model the other options describe, fused with the frozen language
    model of the checkpoint (built from the checkpoint's own options over this run's target vocabulary); the fused
    distribution is ``log_softmax(tm_logits + log p_lm)`` in training, scoring and search.
    (reference: onmt/model_factory.py:913-935, onmt/legacy/FusionNetwork/Models.py:10-72)"""
    import copy

    import torch

    from ..options import backward_compatible
    from ..train.checkpoint import load_model_state
    from .legacy import FusionNetwork
    path = getattr(opt, "lm_checkpoint", "")
    if not path:
        raise ValueError("-fusion needs -lm_checkpoint (a checkpoint written by train_language_model.py)")
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    lm_opt = backward_compatible(ckpt["opt"])
    lm_name = getattr(lm_opt, "model", "transformer_xl_lm")
    lm = _REGISTRY[lm_name if lm_name in ("lstm_lm",) else "transformer_xl_lm"](lm_opt, dicts)
    load_model_state(lm, ckpt["model"])
    tm_opt = copy.copy(opt)
    tm_opt.fusion = False
    tm = build_model(tm_opt, dicts, remove_pretrain)
    return FusionNetwork(tm, lm)


def build_language_model(opt, dicts):
    _load_builders()
    return _REGISTRY["transformer_xl_lm"](opt, dicts)


def build_classifier(opt, dicts):
    _load_builders()
    return _REGISTRY["classifier"](opt, dicts)


def init_model_parameters(model, opt):
    """Re-initialise a freshly built model the way ``-init`` / ``-init_embedding`` / ``-param_init`` ask for
    (reference: onmt/model_factory.py:734-872): ``-init normal`` draws matrices from N(0, 2 / (fan_in + fan_out)),
    ``-init uniform`` uses Xavier-uniform (or U(-param_init, param_init) when ``-param_init`` is set below 0.1 on
    purpose); embeddings are N(0, d^-0.5) (``normal``), N(0, 0.01) (``fixed``) or U(-d^-0.5, d^-0.5) (``uniform``);
    biases start at zero and LayerNorm at (1, 0).  With the default options the models' own construction-time
    initialisation already is this scheme, so the call only acts when an option departs from its default."""
    import math
    import torch
    import torch.nn as nn
    from .layers import Embedding, LayerNorm, Linear
    init = getattr(opt, "init", "normal")
    init_emb = getattr(opt, "init_embedding", "normal")
    param_init = float(getattr(opt, "param_init", 0.1))
    if init == "normal" and init_emb == "normal" and param_init == 0.1:
        return model
    d = int(getattr(opt, "model_size", 512))
    std_emb = d ** -0.5 if not getattr(opt, "rezero", False) else 0.05
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, (Linear, nn.Linear)):
                w = m.weight
                if init == "uniform":
                    if param_init != 0.1:
                        nn.init.uniform_(w, -param_init, param_init)
                    else:
                        nn.init.xavier_uniform_(w)
                else:
                    nn.init.normal_(w, 0.0, math.sqrt(2.0 / (w.shape[0] + w.shape[1])))
                if getattr(m, "bias", None) is not None:
                    m.bias.zero_()
            elif isinstance(m, (Embedding, nn.Embedding)):
                if init_emb == "normal":
                    nn.init.normal_(m.weight, 0.0, std_emb)
                elif init_emb == "fixed":
                    nn.init.normal_(m.weight, 0.0, 0.01)
                else:
                    nn.init.uniform_(m.weight, -std_emb, std_emb)
            elif isinstance(m, (LayerNorm, nn.LayerNorm)):
                m.weight.fill_(1.0)
                m.bias.zero_()
    return model


def optimize_model(model, distributed: bool = False):
    """Projections are created fused (qkv / kv); nothing to convert."""
    return model


_FREEZE_RULES = (
    # option, (substrings of parameter names that it freezes; "enc:" / "dec:" restrict to one side)
    ("freeze_encoder", ("enc:",)),
    ("freeze_decoder", ("dec:",)),
    ("freeze_embedding", ("embed.", "generator.", "word_lut")),
    ("freeze_encoder_self_attn", ("enc:.attn.", "enc:.attn_norm.")),
    ("freeze_encoder_ffn", ("enc:.ffn.", "enc:.ffn_norm.", "enc:.mcr_ffn.")),
    ("freeze_decoder_self_attn", ("dec:.self_attn.", "dec:.self_norm.")),
    ("freeze_decoder_ffn", ("dec:.ffn.", "dec:.ffn_norm.", "dec:.mid_ffn.", "dec:.mcr_ffn.")),
    ("freeze_cross_attention", ("dec:.cross_attn.", "dec:.cross_norm.")),
)


def apply_freeze_options(model, opt) -> int:
    """``-freeze_encoder``, ``-freeze_decoder``, ``-freeze_embedding`` and the per-sub-layer variants: switch off the
    gradients of the named parameter groups (reference: onmt/model_factory.py:333-377 and the ``freeze_*`` checks in
    the wav2vec2 / mBART wrappers).  Returns the number of parameters frozen."""
    frozen = 0
    for flag, patterns in _FREEZE_RULES:
        if not getattr(opt, flag, False):
            continue
        for name, p in model.named_parameters():
            side = "enc:" if name.startswith("encoder.") else ("dec:" if name.startswith("decoder.") else "")
            for pat in patterns:
                if pat.startswith(("enc:", "dec:")):
                    if side != pat[:4] or pat[4:] not in name:
                        continue
                elif pat not in name:
                    continue
                if p.requires_grad:
                    p.requires_grad_(False)
                    frozen += p.numel()
                break
    return frozen


def load_pretrained_parts(model, opt, dicts=None):
    """Pretrained sub-modules named on the command line (see ``models/pretrained_io.py``)."""
    from .pretrained_io import load_pretrained_parts as _load
    return _load(model, opt, dicts)


_loaded = [False]


def _load_builders():
    if _loaded[0]:
        return
    _loaded[0] = True
    from . import transformer as _t

    @register("transformer", "stochastic_transformer")
    def _transformer(opt, dicts):
        return _t.Transformer(opt, dicts)

    import importlib
    for mod in ("pretrained", "relative_transformer", "conformer", "lstm", "transformer_xl", "classifier", "multilingual",
                "research", "legacy"):
        try:
            m = importlib.import_module("." + mod, __package__)
        except ModuleNotFoundError as exc:
            if exc.name and exc.name.endswith(mod):
                continue
            raise
        reg = getattr(m, "register_builders", None)
        if reg is not None:
            reg(register)
