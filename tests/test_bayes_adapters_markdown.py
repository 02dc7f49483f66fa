"""Bayes-by-backprop weight generator, scale-mixture prior, row-indexed adapters and the Markdown option listing."""
import math

import pytest
import torch

from nmtgminor_b200.modules.adapters import EfficientAdapter
from nmtgminor_b200.modules.bayesian import BayesianWeight, Gaussian, ScaleMixtureGaussian


def test_gaussian_and_mixture_log_prob():
    mu, rho = torch.tensor([0.5, -1.0]), torch.tensor([0.0, 1.0])
    g = Gaussian(mu, rho)
    w = torch.tensor([0.2, 0.3])
    want = torch.distributions.Normal(mu, torch.nn.functional.softplus(rho)).log_prob(w).sum()
    assert torch.allclose(g.log_prob(w), want, atol=1e-6)
    assert torch.equal(g.sample(stochastic=False), mu)
    prior = ScaleMixtureGaussian(0.25, 1.0, 0.1)
    n1, n2 = torch.distributions.Normal(0, 1.0), torch.distributions.Normal(0, 0.1)
    want = torch.log(0.25 * n1.log_prob(w).exp() + 0.75 * n2.log_prob(w).exp()).sum()
    assert torch.allclose(prior.log_prob(w), want, atol=1e-5)


@pytest.mark.parametrize("prior", ["standard_normal", "mixture"])
def test_bayesian_weight_gradients_match_autograd(prior):
    torch.manual_seed(0)
    model = torch.nn.Linear(5, 3)
    bw = BayesianWeight(model.parameters(), prior=prior)
    x, y = torch.randn(7, 5), torch.randn(7, 3)
    bw.zero_grad()
    bw.forward(training=True)
    loss = ((model(x) - y) ** 2).sum()
    loss.backward()
    bw.backward()
    kl = bw.kl_divergence(accumulate=True, weight=0.1)
    # the same computation inside autograd
    mean, rho = bw.mean.detach().clone().requires_grad_(True), bw.rho.detach().clone().requires_grad_(True)
    sigma = torch.nn.functional.softplus(rho)
    w = mean + sigma * bw.eps
    W, b = w[:15].view(3, 5), w[15:]
    ref = ((x @ W.t() + b - y) ** 2).sum()
    if prior == "standard_normal":
        ref_kl = 0.5 * (sigma ** 2 + mean ** 2 - 1 - 2 * torch.log(sigma)).sum()
    else:
        ref_kl = Gaussian(mean, rho).log_prob(w) - ScaleMixtureGaussian().log_prob(w)
    (ref + 0.1 * ref_kl).backward()
    assert torch.allclose(kl, ref_kl.detach(), rtol=1e-5)
    assert torch.allclose(bw.mean.grad, mean.grad, atol=1e-4, rtol=1e-4)
    assert torch.allclose(bw.rho.grad, rho.grad, atol=1e-4, rtol=1e-4)
    bw.forward(training=False)
    assert torch.equal(model.weight.detach().reshape(-1), bw.mean.detach()[:15])


def test_bayesian_weight_on_flat_buffers():
    flat, grad = torch.randn(12), torch.randn(12)
    bw = BayesianWeight([], flat=flat, flat_grad=grad)
    before = flat.clone()
    bw.forward(training=True)
    assert not torch.equal(flat, before) and (flat - before).abs().max() < 0.2      # sigma = softplus(-5..-4)
    bw.backward()
    assert torch.equal(bw.mean.grad, grad)


def test_efficient_adapter_rows():
    torch.manual_seed(0)
    ad = EfficientAdapter(3, 16, 4, "gelu")
    x = torch.randn(5, 16)
    assert torch.equal(ad(x, 1), x)                     # zero up-projection: identity at initialisation
    with torch.no_grad():
        ad.up_weight[1].normal_()
    y = ad(x, 1)
    assert not torch.equal(y, x) and torch.equal(ad(x, 0), x)
    h = torch.nn.functional.gelu(torch.nn.functional.layer_norm(x, (16,)) @ ad.down_weight[1].view(4, 16).t())
    assert torch.allclose(y, x + h @ ad.up_weight[1].view(16, 4).t(), atol=1e-5)
    assert all(getattr(p, "adapter", False) for p in ad.parameters())
    y.sum().backward()
    assert ad.up_weight.grad[0].abs().sum() == 0 and ad.up_weight.grad[1].abs().sum() > 0


def test_markdown_help(capsys):
    from nmtgminor_b200.options import make_parser, make_translate_parser
    for make, flag in ((make_parser, "-save_model"), (make_translate_parser, "-beam_size")):
        with pytest.raises(SystemExit):
            make().parse_args(["-md"])
        out = capsys.readouterr().out
        assert "* **%s" % flag in out and out.lstrip().startswith("#")
