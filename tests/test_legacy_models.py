"""The older model zoo: every family builds, trains a step and decodes; the wiring that defines each one is checked."""
import pytest
import torch

from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.models.layers import PackedSeqs
from nmtgminor_b200.models.legacy import (DynamicLinearCombination, FusionNetwork, LSTMLanguageModel, _join_source_target,
                                          layer_major_bank)
from nmtgminor_b200.options import default_options

COMMON = ["-model_size", "64", "-layers", "3", "-n_heads", "2", "-inner_size", "128", "-dropout", "0.0", "-attn_dropout", "0.0",
          "-ffn_activation", "relu", "-label_smoothing", "0.1"]


@pytest.fixture(scope="module")
def dicts():
    d = synthetic_dict(120)
    return {"src": d, "tgt": d}


def _batch():
    return token_budget_batches(120, 4, 10, 60, 1, static=False, padded=True)[0]


@pytest.mark.parametrize("name", ["dlcl_transformer", "parallel_transformer", "fctransformer", "unified_transformer",
                                  "distance_transformer"])
def test_legacy_families_train_and_decode(dicts, name):
    torch.manual_seed(0)
    model = build_model(default_options(["-model", name] + COMMON), dicts)
    batch = _batch()
    out = model(batch)
    assert torch.isfinite(out["loss"]).all()
    out["loss"].backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.parameters())
    model.eval()
    hyps = beam_search(model, batch, BeamConfig(beam_size=2, max_len=5))
    assert len(hyps) == batch.size and all(h[0].tokens for h in hyps)


@pytest.mark.parametrize("name", ["dlcl_transformer", "parallel_transformer", "fctransformer", "unified_transformer"])
def test_incremental_decoding_matches_teacher_forcing(dicts, name):
    """Stepping through the gold prefix gives the same next-token distribution as the training-time forward pass."""
    torch.manual_seed(1)
    model = build_model(default_options(["-model", name] + COMMON), dicts).eval()
    batch = _batch()
    with torch.no_grad():
        full = torch.log_softmax(model(batch, return_logits=True, compute_loss=False)["logprobs"].float(), -1)   # [T, B, V]
        state = model.create_decoder_state(batch, 1)
        tgt_in = batch.get("target_input")
        lengths = batch.packed_target_input().cu.diff()
        for t in range(min(4, int(lengths.min()))):
            step = model.step(tgt_in[:t + 1].t().contiguous(), state)["log_prob"]
            assert torch.allclose(step, full[t], atol=2e-4), (name, t)


def test_dynamic_linear_combination_starts_as_average_and_learns():
    torch.manual_seed(2)
    mix = DynamicLinearCombination(8, 2)
    hist = []
    a, b = torch.randn(5, 8), torch.randn(5, 8)
    mix.push(hist, a)
    assert torch.allclose(mix.pop(hist), a)
    mix.push(hist, b)
    expect = 0.5 * a + 0.5 * mix.norms[1](b)
    assert torch.allclose(mix.pop(hist), expect, atol=1e-6)
    mix.pop(hist).sum().backward()
    assert mix.weight.grad is not None and mix.weight.grad[1, :2].abs().sum() > 0 and mix.weight.grad[0].abs().sum() == 0


def test_layer_major_bank_layout():
    lens = torch.tensor([2, 3])
    toks = torch.zeros(2, 3, dtype=torch.long)
    src = PackedSeqs.from_padded(toks, lens, capacity=7)
    l0 = torch.arange(7.0)[:, None].expand(7, 4).clone()
    l1 = l0 + 100
    bank, seqs = layer_major_bank([l0, l1], src)
    assert seqs.cu.tolist() == [0, 4, 10] and seqs.max_len == 6
    assert bank[:10, 0].tolist() == [0, 1, 100, 101, 2, 3, 4, 102, 103, 104]
    assert bank[10:].abs().sum() == 0


def test_join_source_target_layout():
    src = PackedSeqs.from_padded(torch.tensor([[5, 6, 0], [7, 8, 9]]), torch.tensor([2, 3]))
    tgt = PackedSeqs.from_padded(torch.tensor([[11, 12], [13, 0]]), torch.tensor([2, 1]))
    joint, t_dest, is_src = _join_source_target(src, tgt)
    assert joint.tokens.tolist() == [5, 6, 11, 12, 7, 8, 9, 13]
    assert joint.cu.tolist() == [0, 4, 8] and t_dest.tolist() == [2, 3, 7]
    assert joint.positions.tolist() == [0, 1, 0, 1, 0, 1, 2, 0]
    assert is_src.tolist() == [True, True, False, False, True, True, True, False]


def test_fusion_network_adds_a_frozen_language_model(dicts):
    torch.manual_seed(3)
    opt = default_options(["-model", "transformer"] + COMMON)
    tm = build_model(opt, dicts)
    lm = LSTMLanguageModel(opt, dicts)
    batch = _batch()
    lm_out = lm(batch)
    assert torch.isfinite(lm_out["loss"])
    lm_out["loss"].backward()
    assert lm.rnn.weight_ih_l0.grad.abs().sum() > 0
    fusion = FusionNetwork(tm, lm)
    assert all(not p.requires_grad for p in lm.parameters())
    out = fusion(batch)
    assert torch.isfinite(out["loss"])
    out["loss"].backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in tm.parameters())
    fusion.eval()
    # the fused distribution is log_softmax(tm_logits + log p_lm)
    with torch.no_grad():
        tm_logits = tm(batch, return_logits=True, compute_loss=False)["logprobs"].float()
        expect = torch.log_softmax(tm_logits + lm.log_probs(batch.get("target_input")), -1)
        state = fusion.create_decoder_state(batch, 1)
        step0 = fusion.step(batch.get("target_input")[:1].t().contiguous(), state)["log_prob"]
    assert torch.allclose(step0, expect[0], atol=2e-4)
    hyps = beam_search(fusion, batch, BeamConfig(beam_size=2, max_len=5))
    assert len(hyps) == batch.size


@pytest.mark.parametrize("lm_name", ["transformer_xl_lm", "lstm_lm"])
def test_fusion_flags_build_a_fused_model_from_a_language_model_checkpoint(dicts, tmp_path, lm_name):
    """``-fusion -lm_checkpoint``: the factory loads the language model with its own options and freezes it."""
    torch.manual_seed(4)
    lm_opt = default_options(["-model", lm_name, "-model_size", "32", "-layers", "1", "-n_heads", "2", "-inner_size", "64",
                              "-dropout", "0.0", "-attn_dropout", "0.0"])
    lm = build_model(lm_opt, dicts)
    ckpt = str(tmp_path / "lm.pt")
    torch.save({"model": lm.state_dict(), "opt": lm_opt, "dicts": dicts}, ckpt)
    with pytest.raises(ValueError, match="lm_checkpoint"):
        build_model(default_options(["-model", "transformer", "-fusion"] + COMMON), dicts)
    fused = build_model(default_options(["-model", "transformer", "-fusion", "-lm_checkpoint", ckpt] + COMMON), dicts)
    assert isinstance(fused, FusionNetwork) and all(not p.requires_grad for p in fused.lm_model.parameters())
    for (k, a), b in zip(lm.state_dict().items(), fused.lm_model.state_dict().values()):
        assert torch.equal(a, b), k
    batch = _batch()
    out = fused(batch)
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and any(p.grad is not None and p.grad.abs().sum() > 0 for p in fused.tm_model.parameters())
    fused.eval()
    with torch.no_grad():
        # the language model's prefix distribution equals its training-time forward pass
        log_lm = fused.lm_model.log_probs(batch.get("target_input"))
        tm_logits = fused.tm_model(batch, return_logits=True, compute_loss=False)["logprobs"].float()
        state = fused.create_decoder_state(batch, 1)
        step0 = fused.step(batch.get("target_input")[:1].t().contiguous(), state)["log_prob"]
    assert torch.allclose(log_lm.exp().sum(-1), torch.ones_like(log_lm[..., 0]), atol=1e-4)
    assert torch.allclose(step0, torch.log_softmax(tm_logits + log_lm, -1)[0], atol=2e-4)
    hyps = beam_search(fused, batch, BeamConfig(beam_size=2, max_len=5))
    assert len(hyps) == batch.size
