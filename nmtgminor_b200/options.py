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


# ---------------------------------------------------------------------------------------------------------------
# what every training flag does here: consumed by code, accepted without effect (and why), or refused
# ---------------------------------------------------------------------------------------------------------------
# Flags that select between a fused and an unfused implementation in the reference.  Here the fused kernels are the
# only path on a GPU and the PyTorch restatement the only path on a CPU, so the switches have nothing to choose.
ALWAYS_ON_FLAGS = {
    "fast_xentropy": "the fused label-smoothed cross-entropy kernel is always used on a GPU",
    "fast_xattention": "encoder-decoder attention always runs on the tcgen05 attention kernels",
    "fast_self_attention": "self-attention always runs on the tcgen05 attention kernels",
    "fast_feed_forward": "feed-forward blocks always run as GEMMs with fused epilogues",
    "fused_ffn": "feed-forward blocks always run as GEMMs with fused epilogues",
    "flatten_parameters": "parameters always live in one flat buffer (parallel/flat.py)",
    "zeror_optim": "optimiser state is always sharded across the data-parallel ranks (parallel/sharded.py)",
    "fast_factorize": "factorised weights always go through the GEMM kernels (the same product as the reference's fused form)",
}

# Flags that the reference parses and never reads (checked by grepping its sources): accepted for command-line
# compatibility, without effect there or here.
NO_EFFECT_IN_REFERENCE = {
    "dr_alpha", "dr_beta", "attribute_size", "noam_step_interval", "factorizing_step", "input_feature_size",
    "mfw_atb_rank_scale", "freezing_steps", "debugging", "enc_pretrain_hidden_size", "enc_pretrain_word_dropout",
    "enc_pretrain_attn_dropout", "mutual_modality_training",
    # the trainers add opt.contrastive_loss_coeff * outputs['contrastive_loss'], but no model of the reference ever puts
    # that key into its outputs (the speech models set the term to 0 and leave the assignment commented out)
    "contrastive_loss_coeff",
    # parsed by the training script but never handed to a data set (frames are stacked at preprocessing, or with -concat)
    "reshape_speech",
    # only named in commented-out code of the relative Transformer layers
    "bottleneck_size",
    # parsed into a per-data-set dictionary and handed to Dataset(dataset_factor=...), which never reads it
    "dataset_factors",
    # written to onmt.constants.residual_type; every reader of that constant is commented out
    "residual_type",
}

# Flags whose feature is not built: giving one a value other than its default stops the run instead of silently
# training a different model.
UNSUPPORTED_FLAGS = {
    "stream_context": "streaming context selection",
    "weight_norm": "weight-normalised linear layers",
    "extra_context_size": "extra streaming context",
    "flex_factorize": "flexible-rank factorised weights",
    "sub_encoder": "text sub-encoders behind the speech encoder",
    "enc_stacked_pretrained_model": "stacked pretrained encoders",
    "load_pretrained_classifier": "pretrained classifier heads",
    "wav2vec2_quantize": "the wav2vec 2.0 quantiser inside the translation models (models/w2vbert.py has the quantiser)",
    "wav2vec2_dual_output": "dual-output wav2vec 2.0 encoders",
    "cache_encoder_output": "cached encoder outputs (the reference's own caching pass stops at a debugger breakpoint, "
                            "onmt/train_utils/mp_trainer.py:1549)",
    "use_memory": "the n-gram memory decoder",
    "freeze_baseline_decoder": "the n-gram memory decoder",
    "memory_size_max": "the n-gram memory decoder",
    "encoder_layers_memory": "the n-gram memory decoder",
    "decoder_layers_memory": "the n-gram memory decoder",
    "pos_emb_type": "position-embedding variants of the legacy speech Transformer",
    "char_ctc": "character-level CTC targets",
    "cache_dir": "cached encoder outputs (see -cache_encoder_output)",
    "memory_loss_coeff": "the n-gram memory decoder",
}


def _flag_defaults():
    return {row[0]: (row[1], row[2]) for row in list(TRAIN_FLAGS) + list(EXTRA_TRAIN_FLAGS)}


def unsupported_flags_in(opt):
    """[(flag, value, what)] for every unsupported flag that ``opt`` sets to something other than its default."""
    defaults = _flag_defaults()
    bad = []
    for name, what in UNSUPPORTED_FLAGS.items():
        if not hasattr(opt, name) or name not in defaults:
            continue
        kind, default = defaults[name]
        value = getattr(opt, name)
        if kind == "flag":
            if value:
                bad.append((name, value, what))
        elif value != default and not (value in (None, "", [], 0, 0.0) and default in (None, "", [], 0, 0.0)):
            bad.append((name, value, what))
    return bad


def validate_model_options(opt) -> None:
    """Refuse option values whose feature this build does not have (see ``UNSUPPORTED_FLAGS``)."""
    bad = unsupported_flags_in(opt)
    if bad:
        raise NotImplementedError("not supported by this build: " + "; ".join("-%s %r (%s)" % b for b in bad))
