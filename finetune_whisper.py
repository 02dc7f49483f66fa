#!/usr/bin/env python
"""Fine-tune a Whisper-style speech model with adapters, parameter averaging and / or a teacher.

    python finetune_whisper.py -data corpus -data_format scp -dec_config_file whisper.json -load_from whisper.pt \\
           [-lora_rank 8 -lora_alpha 16] [-ema -ema_decay 0.999] [-teacher teacher.pt -distill_alpha 0.5] [usual training flags]

Takes the flags of ``train_distributed.py``; ``-model`` defaults to ``whisper``.  LoRA freezes the loaded weights and
trains rank-r adapters on the attention projections (optimiser state exists only for the adapters); ``-ema`` keeps an
averaged copy of the parameters that is used for validation and saved; ``-teacher`` adds the distillation term.
(reference: the Hugging Face ``Seq2SeqTrainer`` based scripts under whisper/, here on this framework's trainer)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None):
    import train_distributed as td
    from nmtgminor_b200.models import factory
    from nmtgminor_b200.options import make_parser
    from nmtgminor_b200.train import finetune as ft

    argv = list(sys.argv[1:] if argv is None else argv)
    if "-model" not in argv:
        argv += ["-model", "whisper"]
    opt = make_parser().parse_args(argv)
    rank, alpha = int(getattr(opt, "lora_rank", 0) or 0), float(getattr(opt, "lora_alpha", 16.0))
    teacher_path = getattr(opt, "teacher", "")
    # the adapters are applied here; the trainer must not see the flag again
    if "-lora_rank" in argv:
        i = argv.index("-lora_rank")
        del argv[i:i + 2]
    original_build = factory.build_model

    def build_with_adapters(o, dicts, *a, **kw):
        model = original_build(o, dicts, *a, **kw)
        if getattr(o, "load_from", ""):
            from nmtgminor_b200.train.checkpoint import load_checkpoint, load_model_state
            load_model_state(model, load_checkpoint(o.load_from)["model"])
        if rank > 0:
            replaced = ft.apply_lora(model, r=rank, alpha=alpha)
            print("[INFO] LoRA adapters on %d projections" % len(replaced), flush=True)
        if teacher_path:
            from nmtgminor_b200.train.checkpoint import load_checkpoint, load_model_state
            ck = load_checkpoint(teacher_path)
            teacher = original_build(ck["opt"], ck["dicts"])
            load_model_state(teacher, ck["model"])
            model = ft.DistillationWrapper(model, teacher, getattr(o, "distill_alpha", 0.5), getattr(o, "distill_temperature", 2.0))
        return model

    factory.build_model = build_with_adapters
    import nmtgminor_b200.train.trainer as trainer_mod
    trainer_mod.build_model = build_with_adapters
    try:
        td.cli_main(argv)
    finally:
        factory.build_model = original_build
        trainer_mod.build_model = original_build


if __name__ == "__main__":
    main()
