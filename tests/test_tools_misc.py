import torch

from nmtgminor_b200.tools.kmeans import KMeans, learn_kmeans, quantize
from nmtgminor_b200.tools.text import Autoencoder, extract_vocab, normalize_text, train_autoencoder


def test_kmeans_recovers_separated_clusters():
    torch.manual_seed(0)
    centres = torch.tensor([[0.0, 0.0], [10.0, 0.0], [0.0, 10.0]])
    x = torch.cat([c + 0.1 * torch.randn(200, 2) for c in centres])
    best = min((learn_kmeans([x[torch.randperm(600)]], 3, epochs=5, seed=s) for s in range(4)), key=lambda k: k.inertia(x))
    assert best.inertia(x) < 0.1
    units = quantize(best, x)
    assert len(set(units[:200])) == 1 and len(set(units)) == 3
    assert quantize(best, x[:200], deduplicate=True) == [units[0]]
    again = KMeans.load(best.state_dict())
    assert torch.equal(again.assign(x), best.assign(x))


def test_text_tools_and_autoencoder():
    assert extract_vocab(["b a a", "a c b"], min_count=2) == ["a", "b"]
    assert normalize_text("  “Hello” ,  world !  ", lower=True) == '"hello" , world !'
    assert normalize_text("a, b.", strip_punct=True) == "a b"
    torch.manual_seed(0)
    basis = torch.randn(4, 16)
    states = [torch.tanh(torch.randn(50, 4) @ basis) for _ in range(4)]
    first = Autoencoder(16, 8).loss(states[0]).item()
    ae = train_autoencoder(states, inner_size=8, epochs=40, lr=5e-3)
    assert ae.loss(states[0]).item() < first


def test_speech_benchmark_dry_run(capsys):
    """``bench_speech.py --tiny`` runs both speech configurations through the training engine on the CPU."""
    import importlib.util
    import json
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_speech", os.path.join(root, "bench_speech.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for cfg in ("whisper_large_v2", "wav2vec2_mbart50"):
        mod.main(["--config", cfg, "--tiny", "--steps", "1", "--warmup", "1"])
        line = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1]
        out = json.loads(line)
        assert out["value"] > 0 and out["audio_seconds_per_second"] > 0 and out["loss_per_token_after_warmup"] > 0


def test_preprocess_triangle_and_classify(tmp_path):
    import importlib
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    tri, cls = importlib.import_module("preprocess_triangle"), importlib.import_module("preprocess_classify")
    (tmp_path / "s.txt").write_text("a b c\nd e\n" + "x " * 300 + "\nf g h i\n")
    (tmp_path / "t.txt").write_text("A B\nC\nD\nE F G\n")
    (tmp_path / "a.txt").write_text("u v w\nx\ny\nz z\n")
    (tmp_path / "l.txt").write_text("pos\nneg\npos\nneg\n")
    common = ["-train_src", str(tmp_path / "s.txt"), "-valid_src", str(tmp_path / "s.txt"), "-src_seq_length", "64"]
    out = str(tmp_path / "tri")
    tri.main(common + ["-train_tgt", str(tmp_path / "t.txt"), "-valid_tgt", str(tmp_path / "t.txt"),
                       "-aux_train_tgt", str(tmp_path / "a.txt"), "-aux_valid_tgt", str(tmp_path / "a.txt"), "-save_data", out])
    data = torch.load(out + ".train.pt", weights_only=False)
    tr = data["train"]
    assert len(tr["src"]) == len(tr["tgt"]) == len(tr["aux_tgt"]) == 3            # the 300-word line is dropped on all sides
    aux = data["dicts"]["aux_tgt"]
    assert [aux.get_label(int(i)) for i in tr["aux_tgt"][2][1:-1]] == ["z", "z"]     # aligned with the 4th line
    out2 = str(tmp_path / "cls")
    cls.main(common + ["-train_tgt", str(tmp_path / "l.txt"), "-valid_tgt", str(tmp_path / "l.txt"), "-save_data", out2])
    data = torch.load(out2 + ".train.pt", weights_only=False)
    labels = data["dicts"]["tgt"]
    assert [t.numel() for t in data["train"]["tgt"]] == [1, 1, 1]                     # bare labels, no delimiters
    assert [labels.get_label(int(t[0])) for t in data["train"]["tgt"]] == ["pos", "neg", "neg"]
    try:
        tri.main(common)
        raise AssertionError("missing -aux_train_tgt must be refused")
    except SystemExit:
        pass


def test_rng_state_round_trip():
    import random
    import numpy as np
    from nmtgminor_b200 import ops
    from nmtgminor_b200.train.checkpoint import restore_rng_state, rng_state
    ops.manual_seed(77)
    ops.next_stream()
    state = rng_state()
    want = (random.random(), float(np.random.rand()), torch.rand(3), ops.next_stream())
    random.random(), np.random.rand(), torch.rand(5), ops.manual_seed(5)
    assert restore_rng_state(state) and not restore_rng_state(None)
    got = (random.random(), float(np.random.rand()), torch.rand(3), ops.next_stream())
    assert want[0] == got[0] and want[1] == got[1] and torch.equal(want[2], got[2]) and want[3] == got[3]
    assert ops._Rng.seed == 77


def test_reversible_stacks_pass_a_numerical_gradient_check():
    from nmtgminor_b200.tools.grad_check import check_reversible
    assert check_reversible(8, 2, 1, decoder=False)
    assert check_reversible(8, 1, 2, decoder=True)


def test_nbest_picker_and_pretrained_vocab_extension(tmp_path):
    import torch
    from nmtgminor_b200.tools.checkpoints import main as ckpt_main
    from nmtgminor_b200.tools.nbest import pick_best
    lines = ["a b ||| -1.0 2.0", "c d ||| -0.5 0.0", "e ||| -3.0 1.0", "f g ||| -2.0 9.0"]
    assert list(pick_best(lines, 2, [1.0, 0.0])) == ["c d", "f g"]
    assert list(pick_best(lines, 2, [1.0, 1.0])) == ["a b", "f g"]
    w = {"weights": {"src_embedding.embed_tokens.weight": torch.randn(12, 4), "tgt_embedding.embed_tokens.weight": torch.randn(12, 4),
                     "other": torch.randn(3)}}
    kept = w["weights"]["src_embedding.embed_tokens.weight"][:10].clone()
    torch.save(w, tmp_path / "d.pt")
    (tmp_path / "v.txt").write_text("".join("t%d %d\n" % (i, i) for i in range(10)))
    ckpt_main(["extend-vocab", "-input", str(tmp_path / "d.pt"), "-vocab", str(tmp_path / "v.txt"), "-extra", "5", "-base_size", "10"])
    out = torch.load(str(tmp_path / "d.pt") + ".extend", weights_only=False)["weights"]["src_embedding.embed_tokens.weight"]
    assert out.shape == (15, 4) and torch.equal(out[:10], kept)
    assert all(any(torch.equal(r, k) for k in kept) for r in out[10:])
    assert open(str(tmp_path / "v.txt") + ".extend").read().splitlines()[-1] == "__4__ 14"
