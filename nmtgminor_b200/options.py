"""Command-line options: one table-driven parser per entry point plus checkpoint-compatibility patching.

The flag names, types and defaults are part of the checkpoint format (the parsed namespace is stored in
every checkpoint and used to rebuild the model), so they follow the reference's option set
(options.py:4-657 ``make_parser``, :660-984 ``backward_compatible``; translate.py:20-168;
preprocess.py:27-170).  Here the flags live in declarative tables (``options_spec``) and the three
parsers are generated from them.
"""
from __future__ import annotations

import argparse
from typing import Iterable, Optional, Sequence

from .options_spec import LEGACY_DEFAULTS, PREPROCESS_FLAGS, TRAIN_FLAGS, TRANSLATE_FLAGS

_TYPES = {"int": int, "float": float, "str": str}

# flags of this framework that the reference does not have
EXTRA_TRAIN_FLAGS = [
    ("attn_bias", "flag", False, {}),            # biases on the attention projections of the plain Transformer
    ("cuda_graph", "flag", False, {}),           # capture the training step in a CUDA graph (static capacities)
    ("fused_ddp", "flag", False, {}),            # peer-memory all-reduce fused with the optimiser step
    ("nccl_ddp", "flag", False, {}),             # baseline switch: NCCL all-reduce of the flat gradient buffer
    ("watchdog_timeout", "float", 0.0, {}),      # seconds without a heartbeat before a rank is declared dead
    ("peer_timeout", "float", 0.0, {}),          # milliseconds a kernel waits for a peer GPU before giving up (0: 120 s)
    ("no_cuda_graph", "flag", False, {}),        # run the training step kernel by kernel instead of replaying a graph
    ("trace_nvtx", "flag", False, {}),           # NVTX ranges around layers / buckets
    ("generator_chunk_rows", "int", 0, {}),      # output projection + loss this many rows at a time (logits stay in L2)
    ("fused_conv", "flag", False, {}),
    ("ema_decay", "float", 0.999, {}),           # decay of the parameter average kept with -ema
    ("lora_rank", "int", 0, {}),                 # finetune_whisper.py: rank of the LoRA adapters (0 = full fine-tuning)
    ("lora_alpha", "float", 16.0, {}),
    ("teacher", "str", "", {}),                  # finetune_whisper.py: checkpoint of a teacher model for distillation
    ("distill_alpha", "float", 0.5, {}),
    ("distill_temperature", "float", 2.0, {}),           # speech front-end convolutions through the tcgen05 GEMM (implicit im2col)
]


def _add(parser: argparse.ArgumentParser, rows: Iterable) -> None:
    have = {s for a in parser._actions for s in a.option_strings}
    for name, kind, default, extra in rows:
        flag = "-" + name
        if flag in have:
            continue
        have.add(flag)
        kw = {}
        if kind == "flag":
            kw["action"] = "store_true"
        else:
            kw["type"] = _TYPES[kind]
            kw["default"] = default
            for k in ("nargs", "choices", "required"):
                if k in extra:
                    kw[k] = extra[k]
        parser.add_argument(flag, **kw)


def _md(parser) -> None:
    """``-md``: print the options as Markdown (reference: onmt/markdown.py, wired in train.py / translate.py)."""
    from .utils.markdown import add_md_help_argument
    if not any("-md" in a.option_strings for a in parser._actions):
        add_md_help_argument(parser)


def make_parser(parser: Optional[argparse.ArgumentParser] = None) -> argparse.ArgumentParser:
    """Training parser (``train.py`` / ``train_distributed.py``)."""
    parser = parser or argparse.ArgumentParser(description="train")
    _add(parser, TRAIN_FLAGS)
    _add(parser, EXTRA_TRAIN_FLAGS)
    _md(parser)
    return parser


def make_translate_parser(parser: Optional[argparse.ArgumentParser] = None) -> argparse.ArgumentParser:
    parser = parser or argparse.ArgumentParser(description="translate")
    _add(parser, TRANSLATE_FLAGS)
    _md(parser)
    return parser


def make_preprocess_parser(parser: Optional[argparse.ArgumentParser] = None) -> argparse.ArgumentParser:
    parser = parser or argparse.ArgumentParser(description="preprocess")
    _add(parser, PREPROCESS_FLAGS)
    _md(parser)
    return parser


def default_options(argv: Sequence[str] = ()) -> argparse.Namespace:
    """Namespace with every training flag at its default (``-data`` is filled with a placeholder)."""
    argv = list(argv)
    if "-data" not in argv:
        argv = ["-data", "none"] + argv
    return make_parser().parse_args(argv)


def backward_compatible(opt: argparse.Namespace) -> argparse.Namespace:
    """Fill attributes missing from an older checkpoint's namespace.

    An attribute absent from ``opt`` takes its historical value when one is recorded in
    ``LEGACY_DEFAULTS`` (what the code did before the flag existed), else today's parser default.  A few
    attributes depend on others, as in the reference: ``ffn_dropout`` / ``residual_dropout`` fall back to
    ``dropout``, ``encoder_layers`` to ``-1``.
    """
    defaults = vars(default_options())
    for k, v in LEGACY_DEFAULTS.items():
        if not hasattr(opt, k):
            setattr(opt, k, v)
    for dep in ("ffn_dropout", "residual_dropout"):
        if not hasattr(opt, dep):
            setattr(opt, dep, getattr(opt, "dropout", 0.0))
    for k, v in defaults.items():
        if not hasattr(opt, k):
            setattr(opt, k, v)
    if getattr(opt, "predict_language", 0) is True:
        opt.predict_language = 1
    elif getattr(opt, "predict_language", 0) is False:
        opt.predict_language = 0
    return opt
