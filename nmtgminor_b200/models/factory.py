"""Model factory: ``opt.model`` -> model object.

A registry maps the reference's model names (onmt/model_factory.py:102-731) to builder functions so that
families can be added without touching a central if-chain.  ``build_model`` is the single entry point used
by trainers and translators; ``init_model_parameters`` and ``optimize_model`` exist for API parity (models
initialise themselves and are born with fused projections).
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
    if getattr(opt, "model_type", "") == "lm" or name in ("TransformerXL", "transformer_xl_lm"):
        return _REGISTRY["transformer_xl_lm"](opt, dicts)
    if name not in _REGISTRY:
        raise NotImplementedError("unknown model %r; registered: %s" % (name, sorted(_REGISTRY)))
    model = _REGISTRY[name](opt, dicts)
    aux = dicts.get("aux_tgt") if hasattr(dicts, "get") else None
    if aux is not None and getattr(model, "ctc_linear", None) is not None:
        # "triangle" corpora: the CTC head predicts the auxiliary target (the transcript), which has its own vocabulary
        import torch.nn as nn
        model.ctc_linear = nn.Linear(model.ctc_linear.in_features, aux.size())
        model.ctc_on_aux = True
    return model


def build_language_model(opt, dicts):
    _load_builders()
    return _REGISTRY["transformer_xl_lm"](opt, dicts)


def build_classifier(opt, dicts):
    _load_builders()
    return _REGISTRY["classifier"](opt, dicts)


def init_model_parameters(model, opt):
    """Models of this framework initialise their own weights at construction; kept for API parity."""
    return model


def optimize_model(model, distributed: bool = False):
    """Projections are created fused (qkv / kv); nothing to convert."""
    return model


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
