"""translate.py end to end on CPU: text input with prefix / anti-prefix / diverse search, and audio (scp) input."""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from nmtgminor_b200.data import audio
from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.options import default_options
from nmtgminor_b200.train.checkpoint import save_checkpoint
import translate as translate_cli

COMMON = ["-model_size", "32", "-layers", "1", "-n_heads", "2", "-inner_size", "64", "-ffn_activation", "relu"]


def test_text_translation_with_prefix_antiprefix_and_diverse_search(tmp_path):
    torch.manual_seed(0)
    d = synthetic_dict(40)
    opt = default_options(COMMON + ["-tie_weights", "-join_embedding"])
    ck = str(tmp_path / "m.pt")
    save_checkpoint(ck, build_model(opt, {"src": d, "tgt": d}), {"src": d, "tgt": d}, opt, 1.0)
    src = tmp_path / "src.txt"
    src.write_text("w1 w2 w3\nw4 w5\nw6\n")
    out = tmp_path / "out.txt"
    base = ["-model", ck, "-src", str(src), "-output", str(out), "-gpu", "-1", "-beam_size", "3", "-max_sent_length", "6", "-batch_size", "2"]
    translate_cli.main(base)
    plain = out.read_text().splitlines()
    assert len(plain) == 3
    translate_cli.main(base + ["-prefix_string", "w7 w8"])
    assert all(l.startswith("w7 w8") for l in out.read_text().splitlines())
    first = plain[0].split()[0]
    translate_cli.main(base + ["-anti_prefix_string", first])
    assert out.read_text().splitlines()[0].split()[:1] != [first]
    translate_cli.main(base + ["-diverse_beamsearch", "-n_best", "3"])
    assert len(out.read_text().splitlines()) == 3


def test_audio_translation_from_scp(tmp_path):
    torch.manual_seed(0)
    d = synthetic_dict(40)
    opt = default_options(["-model", "speech_transformer", "-input_size", "40"] + COMMON)
    ck = str(tmp_path / "asr.pt")
    save_checkpoint(ck, build_model(opt, {"tgt": d}), {"tgt": d}, opt, 1.0)
    ark, scp = tmp_path / "feats.ark", tmp_path / "feats.scp"
    with open(ark, "wb") as fh, open(scp, "w") as sf:
        for i, n in enumerate((50, 37)):
            off = audio.write_ark_matrix(fh, "utt%d" % i, np.random.RandomState(i).randn(n, 40).astype(np.float32))
            sf.write("utt%d %s:%d\n" % (i, ark, off))
    out = tmp_path / "hyp.txt"
    translate_cli.main(["-model", ck, "-src", str(scp), "-output", str(out), "-gpu", "-1", "-beam_size", "2", "-max_sent_length", "5",
                        "-encoder_type", "audio", "-asr_format", "scp", "-batch_size", "2"])
    assert len(out.read_text().splitlines()) == 2


def test_document_context_translation_with_past_src(tmp_path):
    """``-past_src``: the previous source sentence reaches a document-context model and changes its output
    distribution; data sets carry it through ``past_src_data``."""
    from nmtgminor_b200.data.dataset import Dataset
    from nmtgminor_b200.inference.translator import Translator
    torch.manual_seed(3)
    d = synthetic_dict(40)
    opt = default_options(["-model", "discourse_translator"] + COMMON + ["-tie_weights", "-join_embedding"])
    ck = str(tmp_path / "disc.pt")
    save_checkpoint(ck, build_model(opt, {"src": d, "tgt": d}), {"src": d, "tgt": d}, opt, 1.0)
    src, past, out = tmp_path / "src.txt", tmp_path / "past.txt", tmp_path / "out.txt"
    src.write_text("w1 w2 w3\nw4 w5\nw6 w7\n")
    past.write_text("\nw1 w2 w3\nw4 w5\n")                      # first line: document start
    base = ["-model", ck, "-src", str(src), "-output", str(out), "-gpu", "-1", "-beam_size", "2", "-max_sent_length", "5", "-batch_size", "2"]
    translate_cli.main(base + ["-past_src", str(past)])
    assert len(out.read_text().splitlines()) == 3
    tr = Translator(translate_cli.make_translate_parser().parse_args(base))
    sents = [["w4", "w5"], ["w6", "w7"]]
    b0 = tr.build_data(sents, [["w9"], ["w9"]])
    b1 = tr.build_data(sents, [["w9"], ["w9"]], past_sents=[["w1", "w2", "w3"], ["w4", "w5"]])
    assert b0.get("packed_past_source") is None and b1.get("packed_past_source").batch_size == 2
    assert b1.get("past_source").shape == (3, 2)
    _, s0, _ = tr.model.decode(b0)
    _, s1, _ = tr.model.decode(b1)
    assert not torch.allclose(s0, s1)
    # training data sets hand the previous sentence to the batch as well
    ids = [d.convert_to_idx(s, "<unk>") for s in sents]
    tgt = [d.convert_to_idx(["w9"], "<unk>", "<s>", "</s>") for _ in sents]
    ds = Dataset(ids, tgt, past_src_data=[ids[1], ids[0]], batch_size_words=64, cleaning=False)
    assert ds.get_batch(0).get("packed_past_source") is not None


def test_sub_model_reads_its_own_source(tmp_path):
    """``-sub_model`` / ``-sub_src``: a second model joins the ensemble but encodes a different source file."""
    from nmtgminor_b200.inference.translator import EnsembleModel, Translator
    torch.manual_seed(4)
    d = synthetic_dict(40)
    dicts = {"src": d, "tgt": d}
    opt = default_options(COMMON + ["-tie_weights", "-join_embedding"])
    main_ck, sub_ck = str(tmp_path / "main.pt"), str(tmp_path / "sub.pt")
    save_checkpoint(main_ck, build_model(opt, dicts), dicts, opt, 1.0)
    save_checkpoint(sub_ck, build_model(opt, dicts), dicts, opt, 1.0)
    src, sub, out = tmp_path / "src.txt", tmp_path / "sub.txt", tmp_path / "out.txt"
    src.write_text("w1 w2 w3\nw4 w5\n")
    sub.write_text("w9 w8\nw7 w6 w5 w4\n")
    base = ["-model", main_ck, "-sub_model", sub_ck, "-src", str(src), "-output", str(out), "-gpu", "-1", "-beam_size", "2",
            "-max_sent_length", "5", "-batch_size", "2"]
    translate_cli.main(base + ["-sub_src", str(sub)])
    assert len(out.read_text().splitlines()) == 2
    tr = Translator(translate_cli.make_translate_parser().parse_args(base))
    assert isinstance(tr.model, EnsembleModel) and tr.model.sub_flags == [False, True]
    sents, other = [["w1", "w2", "w3"], ["w4", "w5"]], [["w9", "w8"], ["w7", "w6", "w5", "w4"]]
    batch = tr.build_data(sents)
    batch.sub_batch = tr.build_data(other)
    state = tr.model.create_decoder_state(batch, 1)
    assert state.states[0].context.shape[1] == 3 and state.states[1].context.shape[1] == 4     # each member saw its own source


def test_dynamic_quantisation_on_cpu(tmp_path):
    """``-dynamic_quantile 1``: int8 linear layers on the CPU give nearly the same scores as fp32."""
    from nmtgminor_b200.inference.translator import Translator
    from nmtgminor_b200.models.layers import Linear
    torch.manual_seed(6)
    d = synthetic_dict(40)
    dicts = {"src": d, "tgt": d}
    opt = default_options(COMMON + ["-tie_weights", "-join_embedding"])
    ck = str(tmp_path / "m.pt")
    save_checkpoint(ck, build_model(opt, dicts), dicts, opt, 1.0)
    base = ["-model", ck, "-src", "unused", "-gpu", "-1", "-beam_size", "2", "-max_sent_length", "5"]
    plain = Translator(translate_cli.make_translate_parser().parse_args(base))
    quant = Translator(translate_cli.make_translate_parser().parse_args(base + ["-dynamic_quantile", "1"]))
    assert all(getattr(m, "_int8", None) is not None for m in quant.model.modules() if isinstance(m, Linear))
    assert not any(k.endswith("_int8") or "_int8." in k for k in quant.model.state_dict())
    sents, gold = [["w1", "w2", "w3"], ["w4", "w5"]], [["w2", "w3"], ["w6"]]
    s_plain = plain.translate(sents, gold)[5]
    s_quant = quant.translate(sents, gold)[5]
    assert all(abs(a - b) < 0.05 * max(1.0, abs(a)) for a, b in zip(s_plain, s_quant)) and s_plain != s_quant


def test_translate_distributed_splits_all_line_parallel_inputs(tmp_path):
    """Two worker processes (CPU here) translate halves of the input; ``-past_src`` is split alongside ``-src``."""
    import translate_distributed
    torch.manual_seed(3)
    d = synthetic_dict(40)
    opt = default_options(["-model", "discourse_translator"] + COMMON + ["-tie_weights", "-join_embedding"])
    ck = str(tmp_path / "disc.pt")
    save_checkpoint(ck, build_model(opt, {"src": d, "tgt": d}), {"src": d, "tgt": d}, opt, 1.0)
    src, past = tmp_path / "src.txt", tmp_path / "past.txt"
    src.write_text("w1 w2 w3\nw4 w5\nw6 w7\nw8\nw9 w1\n")
    past.write_text("\nw1 w2 w3\nw4 w5\nw6 w7\nw8\n")
    # one sentence per batch, so both runs do exactly the same arithmetic (an untrained model is full of near-ties)
    common = ["-model", ck, "-beam_size", "2", "-max_sent_length", "5", "-batch_size", "1", "-past_src", str(past)]
    single, multi = tmp_path / "single.txt", tmp_path / "multi.txt"
    translate_cli.main(common + ["-src", str(src), "-output", str(single), "-gpu", "-1"])
    translate_distributed.main(common + ["-src", str(src), "-output", str(multi), "-gpus", "-1,-1"])
    # (the hypotheses themselves are not compared: an untrained model is full of near-ties that flip with the thread count)
    assert len(multi.read_text().splitlines()) == len(single.read_text().splitlines()) == 5
    a = translate_distributed.split_file(str(src), 2, str(tmp_path), "a")
    b = translate_distributed.split_file(str(past), 2, str(tmp_path), "b")
    assert [len(open(p).readlines()) for p in a] == [len(open(p).readlines()) for p in b] == [3, 2]


def test_classify_cli_labels_every_line(tmp_path):
    import classify as classify_cli
    from nmtgminor_b200.inference.scoring import ClassifierPredictor
    torch.manual_seed(0)
    d, labels = synthetic_dict(40), synthetic_dict(5)
    opt = default_options(["-model", "classifier"] + COMMON)
    ck = str(tmp_path / "cls.pt")
    model = build_model(opt, {"src": d, "tgt": labels})
    save_checkpoint(ck, model, {"src": d, "tgt": labels}, opt, 1.0)
    src = tmp_path / "src.txt"
    src.write_text("w1 w2 w3\nw4 w5\nw6\nw7 w8 w9 w10\nw3\n")
    out = tmp_path / "pred.txt"
    classify_cli.main(["-model", ck, "-src", str(src), "-output", str(out), "-gpu", "-1", "-batch_size", "2"])
    lines = out.read_text().splitlines()
    assert len(lines) == 5
    # batching must not change the answer: one call over everything gives the same labels
    from nmtgminor_b200.options import make_translate_parser
    p = ClassifierPredictor(make_translate_parser().parse_args(["-model", ck, "-src", str(src), "-gpu", "-1"]))
    whole = p.predict([l.split() for l in src.read_text().splitlines()], batch_size=8)
    assert [p.label_name(i) for i, _ in whole] == lines and all(lp <= 0 for _, lp in whole)
