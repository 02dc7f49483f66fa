"""CPU (fp32, PyTorch-op path) behaviour of the Transformer: training, checkpoint interchange with the
reference's key names, incremental decoding, beam search."""
import copy
import itertools
import math

import pytest
import torch

from nmtgminor_b200.data.dataset import collate
from nmtgminor_b200.data.synthetic import synthetic_dataset, synthetic_dict, synthetic_pairs
from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search, greedy_search
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.options import default_options
from nmtgminor_b200.train.checkpoint import (load_checkpoint, load_model_state, prune_checkpoints, save_checkpoint,
                                             transformer_from_reference, transformer_to_reference)
from nmtgminor_b200.train.engine import TrainEngine
from nmtgminor_b200.train.optim import Optim, learning_rate_at


def tiny_opt(extra=()):
    return default_options(["-model", "transformer", "-model_size", "64", "-layers", "2", "-n_heads", "2", "-inner_size", "128",
                            "-tie_weights", "-join_embedding", "-ffn_activation", "relu", "-label_smoothing", "0.1", "-optim",
                            "adam", "-learning_rate", "0.002", "-update_method", "regular", "-dropout", "0.0", "-attn_dropout",
                            "0.0", "-emb_dropout", "0.0"] + list(extra))


@pytest.fixture(scope="module")
def setup():
    torch.manual_seed(0)
    d = synthetic_dict(60)
    opt = tiny_opt()
    model = build_model(opt, {"src": d, "tgt": d})
    return opt, d, model


def test_training_reduces_loss(setup):
    opt, d, _ = setup
    torch.manual_seed(1)
    model = build_model(opt, {"src": d, "tgt": d})
    eng = TrainEngine(model, opt, device="cpu")
    ds = synthetic_dataset(64, 60, 4, 9, 200, seed=3)
    first = last = None
    for epoch in range(12):
        for i in range(len(ds)):
            b = ds.get_batch(i)
            loss, _ = eng.train_step(b)
            v = float(loss) / b.tgt_size
            first = v if first is None else first
            last = v
    assert last < first - 0.8, (first, last)


def test_reference_named_checkpoint_roundtrip(setup, tmp_path):
    opt, d, model = setup
    sd = model.state_dict()
    ref_sd = transformer_to_reference(sd)
    assert "encoder.layer_modules.0.multihead.fc_query.function.linear.weight" in ref_sd
    assert "decoder.layer_modules.1.multihead_src.fc_value.function.linear.weight" in ref_sd
    assert "generator.0.linear.weight" in ref_sd and "encoder.word_lut.weight" in ref_sd
    back = transformer_from_reference(ref_sd, sd.keys())
    for k, v in sd.items():
        assert k in back, k
        assert torch.equal(back[k], v.float()), k
    path = str(tmp_path / "m_ppl_3.500000_e1.00.pt")
    optim = Optim(opt)
    optim.set_parameters(model.parameters())
    save_checkpoint(path, model, {"src": d, "tgt": d}, opt, 1.0, optim)
    ck = load_checkpoint(path)
    assert set(ck) >= {"model", "dicts", "opt", "epoch", "itr", "optim", "scaler"}
    fresh = build_model(ck["opt"], ck["dicts"])
    missing, unexpected = load_model_state(fresh, ck["model"])
    assert not unexpected
    for (k, a), (_, b) in zip(model.state_dict().items(), fresh.state_dict().items()):
        assert torch.allclose(a, b), k


def test_prune_checkpoints_keeps_best(tmp_path):
    base = str(tmp_path / "model")
    for ppl, ep in ((9.0, 1), (5.0, 2), (7.0, 3), (6.0, 4)):
        open("%s_ppl_%.6f_e%.2f.pt" % (base, ppl, ep), "w").close()
    kept = prune_checkpoints(base, 2, "ppl")
    assert len(kept) == 2 and "5.000000" in kept[0] and "6.000000" in kept[1]
    import glob
    assert len(glob.glob(base + "_ppl_*")) == 2


def test_incremental_decoding_matches_teacher_forcing(setup):
    opt, d, model = setup
    model.eval()
    src, tgt = synthetic_pairs(4, 60, 3, 8, seed=9)
    batch = collate(src, tgt, round_to=1)
    with torch.no_grad():
        full = model(batch, return_logits=True)["logprobs"]            # [T, B, V] logits
        full = torch.log_softmax(full.float(), -1)
        state = model.create_decoder_state(batch, 1)
        tgt_in = batch.get("target_input").t()                          # [B, T]
        for t in range(tgt_in.shape[1]):
            lp = model.step(tgt_in[:, :t + 1], state)["log_prob"]
            lengths = batch.get("tgt_lengths") - 1
            alive = t < lengths
            assert torch.allclose(lp[alive], full[t][alive], atol=2e-4), "step %d" % t


def _sequence_logprob(model, batch_src, hyp, bos=2):
    tgt = [torch.tensor([bos] + hyp)]
    b = collate(batch_src, tgt, round_to=1)
    out = model(b)
    return -float(out["loss"])


def test_beam_search_finds_the_exhaustive_optimum():
    torch.manual_seed(5)
    d = synthetic_dict(9)                   # 5 real words: exhaustive search is cheap
    opt = tiny_opt(["-label_smoothing", "0.0"])
    model = build_model(opt, {"src": d, "tgt": d})
    model.eval()
    src = [torch.tensor([4, 5, 6, 7])]
    batch = collate(src, None, round_to=1)
    cfg = BeamConfig(beam_size=100, n_best=3, max_len=3, min_len=1)   # wider than every prefix set: exhaustive
    hyps = beam_search(model, batch, cfg)[0]
    # brute force over all sequences of <= 3 content tokens followed by EOS
    best = (-1e9, None)
    with torch.no_grad():
        for L in range(1, 4):
            for seq in itertools.product([1, 2, 4, 5, 6, 7, 8], repeat=L):
                s = _sequence_logprob(model, src, list(seq) + [3])
                if s > best[0]:
                    best = (s, list(seq) + [3])
    assert hyps[0].tokens == best[1], (hyps[0], best)
    assert abs(hyps[0].score - best[0]) < 1e-3
    assert all(hyps[i].score >= hyps[i + 1].score for i in range(len(hyps) - 1))
    assert abs(sum(hyps[0].positional_scores) - hyps[0].score) < 1e-3
    g = greedy_search(model, batch, max_len=3)[0]
    assert g[-1] == 3 or len(g) == 4


def test_beam_constraints():
    torch.manual_seed(6)
    d = synthetic_dict(12)
    model = build_model(tiny_opt(), {"src": d, "tgt": d})
    model.eval()
    src = [torch.tensor([4, 5, 6]), torch.tensor([7, 8])]
    batch = collate(src, None, round_to=1)
    hyps = beam_search(model, batch, BeamConfig(beam_size=3, max_len=6, min_len=4))
    assert all(len(h[0].tokens) >= 5 for h in hyps)                 # >= 4 symbols + EOS
    hyps = beam_search(model, batch, BeamConfig(beam_size=3, max_len=8, min_len=3, no_repeat_ngram_size=1))
    for h in hyps:
        body = h[0].tokens[:-1]
        assert len(set(body)) == len(body)
    prefix = torch.tensor([[9, 10], [11, 0]])
    hyps = beam_search(model, batch, BeamConfig(beam_size=3, max_len=6), prefix_tokens=prefix)
    assert hyps[0][0].tokens[:2] == [9, 10] and hyps[1][0].tokens[0] == 11


def test_learning_rate_schedules():
    opt = default_options(["-update_method", "noam", "-warmup_steps", "100", "-learning_rate", "2.0", "-model_size", "256"])
    init = 256 ** -0.5 * 2.0
    assert math.isclose(learning_rate_at(1, opt, init), init * 100 ** -1.5)
    assert math.isclose(learning_rate_at(100, opt, init), init * 100 ** -0.5)
    assert math.isclose(learning_rate_at(400, opt, init), init * 400 ** -0.5)
    o = Optim(opt)
    assert math.isclose(o.init_lr, init)
    cos = default_options(["-update_method", "cosine", "-warmup_steps", "10", "-learning_rate", "1.0", "-max_step", "110"])
    assert math.isclose(learning_rate_at(5, cos, 1.0), 0.5)
    assert learning_rate_at(60, cos, 1.0) == pytest.approx(0.5, abs=1e-6)
    assert learning_rate_at(110, cos, 1.0) == pytest.approx(0.0, abs=1e-6)
