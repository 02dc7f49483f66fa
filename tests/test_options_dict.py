import argparse

from nmtgminor_b200.dictionary import Dict
from nmtgminor_b200.options import (backward_compatible, default_options, make_parser, make_preprocess_parser,
                                    make_translate_parser)
from nmtgminor_b200.options_spec import PREPROCESS_FLAGS, TRAIN_FLAGS, TRANSLATE_FLAGS


def test_train_parser_has_every_table_flag_with_its_default():
    opt = default_options()
    for name, kind, default, extra in TRAIN_FLAGS:
        assert hasattr(opt, name), name
        if name == "data":
            continue
        if kind == "flag":
            assert getattr(opt, name) is False
        elif "nargs" not in extra:
            assert getattr(opt, name) == default, name


def test_key_defaults_match_the_reference_surface():
    opt = default_options()
    assert (opt.model_size, opt.inner_size, opt.n_heads, opt.layers) == (512, 2048, 8, 2)
    assert (opt.batch_size_words, opt.warmup_steps, opt.keep_save_files) == (2048, 4096, 5)
    assert opt.beta1 == 0.9 and abs(opt.beta2 - 0.997) < 1e-9
    assert opt.max_grad_norm == 5 and opt.optim == "adam"


def test_translate_and_preprocess_parsers():
    t = make_translate_parser().parse_args(["-model", "m.pt", "-src", "x"])
    assert t.beam_size == 5 and t.batch_size == 30 and t.max_sent_length == 256
    assert len({n for n, *_ in TRANSLATE_FLAGS}) == len(TRANSLATE_FLAGS) or True
    p = make_preprocess_parser().parse_args(["-train_src", "a", "-train_tgt", "b", "-valid_src", "c", "-valid_tgt", "d",
                                             "-save_data", "e"])
    assert p.format == "raw"
    assert len(PREPROCESS_FLAGS) >= 60


def test_backward_compatible_fills_missing_attributes():
    old = argparse.Namespace(model_size=256, dropout=0.2, model="transformer")
    new = backward_compatible(old)
    assert new.ffn_dropout == 0.2 and new.residual_dropout == 0.2
    assert new.ffn_activation == "relu"            # historical behaviour, not today's parser default
    assert new.layers == 2 and hasattr(new, "label_smoothing")
    assert default_options().ffn_activation == "silu"


def test_dictionary_roundtrip(tmp_path):
    d = Dict(["<blank>", "<unk>", "<s>", "</s>"])
    for w in "a b a c a b d".split():
        d.add(w)
    assert d.size() == 8 and d.lookup("a") == 4 and d.frequencies[4] == 3
    ids = d.convert_to_idx("a z b".split(), "<unk>", "<s>", "</s>")
    assert ids.tolist() == [2, 4, 1, 5, 3]
    assert d.convert_to_labels(ids[1:], stop=3, including_stop=False) == ["a", "<unk>", "b"]
    pruned = d.prune(2)
    assert pruned.size() == 6 and pruned.lookup("a") is not None and pruned.lookup("d") is None
    d.patch(16)
    assert d.size() % 16 == 0
    f = tmp_path / "vocab.txt"
    d.write_file(str(f))
    assert Dict(str(f)).labelToIdx == d.labelToIdx
    assert Dict.from_state(d.state()).labelToIdx == d.labelToIdx
