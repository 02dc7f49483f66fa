"""Noise-contrastive output layer (alias sampler, NCELinear, NCELoss, model wiring) and the language-model fusion loss."""
import math

import torch

from nmtgminor_b200.data.dataset import collate
from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.modules.nce import AliasSampler, NCELinear, NCELoss, build_unigram_noise
from nmtgminor_b200.options import default_options
from nmtgminor_b200.train.loss import FusionLoss


def test_alias_sampler_follows_the_distribution():
    torch.manual_seed(0)
    p = torch.tensor([0.5, 0.05, 0.2, 0.01, 0.24])
    s = AliasSampler(p)
    draws = s.draw(200000)
    freq = torch.bincount(draws, minlength=5).float() / draws.numel()
    assert torch.allclose(freq, p, atol=5e-3)
    assert s.draw(3, 4).shape == (3, 4)


def test_unigram_noise_from_dictionary():
    d = synthetic_dict(20)
    d.frequencies = {i: (i + 1) for i in range(d.size())}
    p = build_unigram_noise(dictionary=d)
    assert abs(float(p.sum()) - 1) < 1e-6 and p[-1] > p[0] > 0
    assert torch.allclose(build_unigram_noise(vocab_size=8), torch.full((8,), 0.125))


def test_nce_loss_formula_and_learning():
    torch.manual_seed(1)
    V, H, N, K = 50, 16, 64, 8
    noise = build_unigram_noise(torch.arange(1, V + 1).float())
    lin = NCELinear(H, V, noise, K)
    loss_fn = NCELoss(H, V, K, logz=2.0, label_smoothing=0.0, padding_idx=0)
    h = torch.randn(N, H)
    y = torch.randint(1, V, (N,))
    y[:5] = 0                                            # padding rows do not count
    lin.train(); loss_fn.train()
    out = lin(h, y)
    res = loss_fn(out, y)
    # by hand: -log sigma(x_target) - sum log (1 - sigma(x_noise))
    keep = y != 0
    xt = out["scores_model_target"][keep] - 2.0 - out["logprob_noise_target"][keep] - math.log(K)
    xn = out["scores_model_noise"][keep] - 2.0 - out["logprob_noise_noise"][keep] - math.log(K)
    ref = -(torch.nn.functional.logsigmoid(xt).sum() + torch.nn.functional.logsigmoid(-xn).sum())
    assert torch.allclose(res["loss"], ref, rtol=1e-5)
    # evaluation: ordinary cross-entropy over the same weights
    lin.eval(); loss_fn.eval()
    ev = loss_fn(lin(h), y)
    full = torch.nn.functional.cross_entropy((h @ lin.weight.t() + lin.bias)[keep], y[keep], reduction="sum")
    assert torch.allclose(ev["loss"], full, rtol=1e-5)
    # a few NCE steps on a fixed mapping reduce the true cross-entropy
    lin.train(); loss_fn.train()
    opt = torch.optim.Adam(lin.parameters(), lr=0.05)
    before = float(full)
    for _ in range(150):
        opt.zero_grad()
        loss_fn(lin(h, y), y)["loss"].backward()
        opt.step()
    lin.eval()
    after = float(torch.nn.functional.cross_entropy((h @ lin.weight.t() + lin.bias)[keep], y[keep], reduction="sum"))
    assert after < 0.7 * before


def test_model_trains_with_nce_noise():
    torch.manual_seed(0)
    d = synthetic_dict(30)
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-ffn_activation", "relu"])
    opt.nce_noise = 6
    m = build_model(opt, {"src": d, "tgt": d})
    assert m.nce.weight is m.generator.weight
    b = collate([torch.tensor([5, 6, 7])], [torch.tensor([2, 8, 9, 3])], padded=True, packed=True)
    m.train()
    out = m(b)
    out["loss"].sum().backward()
    assert m.generator.weight.grad is not None and float(out["loss"]) > 0
    m.eval()
    with torch.no_grad():
        ev = m(b)
    assert ev["correct"] is not None          # evaluation goes through the ordinary fused cross-entropy


def test_fusion_loss_prenorm():
    torch.manual_seed(0)
    T, B, H, V = 4, 2, 8, 11

    class Side(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.generator = torch.nn.Linear(H, V)

    class Both(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.tm_model, self.lm_model = Side(), Side()

    model = Both()
    tm, lm = torch.randn(T, B, H, requires_grad=True), torch.randn(T, B, H)
    y = torch.randint(1, V, (T, B))
    y[-1, 1] = 0
    fl = FusionLoss(V, 0.0, 0)
    fl.eval()
    res = fl({"tm": {"hidden": tm}, "lm": {"hidden": lm}}, y, model=model, backward=True, normalizer=2.0)
    fused = torch.log_softmax(model.tm_model.generator(tm) + torch.log_softmax(model.lm_model.generator(lm), -1), -1)
    ref = torch.nn.functional.nll_loss(fused.view(-1, V), y.view(-1), ignore_index=0, reduction="sum")
    assert torch.allclose(res["loss"], ref, rtol=1e-5) and res["total"] == T * B - 1
    assert tm.grad is not None and model.lm_model.generator.weight.grad is None
