"""Bayes-by-backprop building blocks: a diagonal Gaussian posterior, the two-component scale-mixture prior, and a
weight generator that keeps a posterior over EVERY parameter of a model.

Reference: onmt/modules/bayes_by_backprop/gaussian.py:10-75 (``Gaussian``, ``ScaleMixtureGaussian``),
onmt/bayesian_weight_generator.py:44-170 (``BayesianWeight``: flatten the parameters, draw ``w = mu + softplus(rho) * eps``
before the forward pass, route ``dL/dw`` to ``mu`` and ``rho`` after the backward pass, KL against the prior).

``BayesianWeight`` works on one flat view of the parameters, which is how this framework stores them anyway: when the
model was flattened by ``parallel/flat.py`` the sampled weights are written into the fp32 master buffer in one call and
the gradient is read from the flat gradient buffer; otherwise a flat copy is scattered to / gathered from the tensors.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch
import torch.nn.functional as F

PI, SIGMA_1, SIGMA_2 = 0.5, math.exp(-0.0), math.exp(-6.0)
_LOG_SQRT_2PI = 0.5 * math.log(2.0 * math.pi)


class Gaussian:
    """Diagonal Gaussian parameterised by ``mu`` and ``rho`` (``sigma = softplus(rho)``)."""

    def __init__(self, mu: torch.Tensor, rho: torch.Tensor):
        self.mu, self.rho = mu, rho

    @property
    def sigma(self) -> torch.Tensor:
        return F.softplus(self.rho)

    def sample(self, stochastic: bool = True, return_log_prob: bool = False, generator=None):
        if not stochastic:
            w = self.mu
        else:
            eps = torch.randn(self.mu.shape, generator=generator, device=self.mu.device, dtype=self.mu.dtype)
            w = self.mu + self.sigma * eps
        return (w, self.log_prob(w)) if return_log_prob else w

    def log_prob(self, w: torch.Tensor) -> torch.Tensor:
        s = self.sigma
        return (-_LOG_SQRT_2PI - torch.log(s) - (w - self.mu) ** 2 / (2 * s ** 2)).sum()


# run-wide prior of the scale mixture, set from the command line by ``configure_prior``
PRIOR = {"pi": PI, "sigma1": SIGMA_1, "sigma2": SIGMA_2}


def configure_prior(opt) -> dict:
    """``-prior_pi``, ``-neg_log_sigma1``, ``-neg_log_sigma2``: mixture weight and the two standard deviations, given as
    negative logarithms (reference: onmt/bayesian_factory.py / onmt/modules/bayes_by_backprop: ``sigma = exp(-x)``)."""
    PRIOR["pi"] = float(getattr(opt, "prior_pi", PI))
    PRIOR["sigma1"] = math.exp(-float(getattr(opt, "neg_log_sigma1", -math.log(SIGMA_1))))
    PRIOR["sigma2"] = math.exp(-float(getattr(opt, "neg_log_sigma2", -math.log(SIGMA_2))))
    return dict(PRIOR)


class ScaleMixtureGaussian:
    """Prior ``pi * N(0, sigma1^2) + (1 - pi) * N(0, sigma2^2)`` (Blundell et al. 2015)."""

    def __init__(self, pi: Optional[float] = None, sigma1: Optional[float] = None, sigma2: Optional[float] = None):
        self.pi = PRIOR["pi"] if pi is None else pi
        self.sigma1 = PRIOR["sigma1"] if sigma1 is None else sigma1
        self.sigma2 = PRIOR["sigma2"] if sigma2 is None else sigma2

    def _component(self, w, sigma):
        return -_LOG_SQRT_2PI - math.log(sigma) - w ** 2 / (2 * sigma ** 2)

    def log_prob(self, w: torch.Tensor) -> torch.Tensor:
        a = self._component(w, self.sigma1) + math.log(self.pi)
        b = self._component(w, self.sigma2) + math.log(1.0 - self.pi)
        return torch.logaddexp(a, b).sum()


class BayesianWeight:
    """Posterior over all parameters of a model, outside autograd.

    Per step: ``forward(training)`` writes a sample (or the mean) into the parameters; the model runs and back-propagates
    as usual; ``backward()`` adds ``dL/dw`` to ``mean.grad`` and ``dL/dw * eps * sigmoid(rho)`` to ``rho.grad`` (the chain
    rule through ``w = mean + softplus(rho) * eps``); ``kl_divergence()`` gives the complexity term and, with
    ``accumulate=True``, adds its gradient too.  ``parameters()`` (mean, rho) is what the optimiser updates.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], prior: str = "standard_normal", flat: Optional[torch.Tensor] = None,
                 flat_grad: Optional[torch.Tensor] = None):
        assert prior in ("standard_normal", "mixture")
        self.params = [p for p in params]
        self.flat, self.flat_grad = flat, flat_grad            # the caller's flat buffers, if the model has them
        n = sum(p.numel() for p in self.params) if flat is None else flat.numel()
        ref = self.params[0] if flat is None else flat
        self.mean = torch.nn.Parameter(self._gather_values().clone())
        self.rho = torch.nn.Parameter(torch.empty(n, device=ref.device, dtype=torch.float32).uniform_(-5.0, -4.0))
        self.mean.grad, self.rho.grad = torch.zeros_like(self.mean), torch.zeros_like(self.rho)
        self.eps = torch.zeros_like(self.mean)
        self.sampled = False
        self.prior_type = prior
        self.prior = ScaleMixtureGaussian() if prior == "mixture" else None

    # -- flat <-> tensors ------------------------------------------------------------------------------------------
    def _gather_values(self) -> torch.Tensor:
        if self.flat is not None:
            return self.flat.detach().float()
        return torch.cat([p.detach().float().reshape(-1) for p in self.params])

    def _gather_grads(self) -> torch.Tensor:
        if self.flat_grad is not None:
            return self.flat_grad.detach().float()
        return torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).detach().float().reshape(-1)
                          for p in self.params])

    def _scatter(self, w: torch.Tensor) -> None:
        if self.flat is not None:
            self.flat.copy_(w)
            return
        o = 0
        for p in self.params:
            p.data.copy_(w[o:o + p.numel()].view_as(p))
            o += p.numel()

    # -- the three calls of a step ---------------------------------------------------------------------------------
    def parameters(self):
        return [self.mean, self.rho]

    def zero_grad(self) -> None:
        self.mean.grad.zero_()
        self.rho.grad.zero_()

    @torch.no_grad()
    def forward(self, training: bool = True, generator=None) -> None:
        if training:
            self.eps.copy_(torch.randn(self.eps.shape, generator=generator, device="cpu" if generator is not None else self.eps.device))
            self._scatter(self.mean + F.softplus(self.rho) * self.eps)
        else:
            self._scatter(self.mean.detach())
        self.sampled = training

    @torch.no_grad()
    def backward(self) -> None:
        g = self._gather_grads()
        self.mean.grad.add_(g)
        if self.sampled:
            self.rho.grad.add_(torch.sigmoid(self.rho) * self.eps * g)

    def kl_divergence(self, accumulate: bool = False, weight: float = 1.0) -> torch.Tensor:
        """KL(q || prior): closed form for the standard normal prior, the one-sample estimate
        ``log q(w) - log p(w)`` at the last drawn ``w`` for the mixture prior."""
        mean, rho = self.mean.detach().requires_grad_(accumulate), self.rho.detach().requires_grad_(accumulate)
        sigma = F.softplus(rho)
        if self.prior_type == "standard_normal":
            kl = 0.5 * (sigma ** 2 + mean ** 2 - 1.0 - 2.0 * torch.log(sigma)).sum()
        else:
            w = mean + sigma * self.eps
            kl = Gaussian(mean, rho).log_prob(w) - self.prior.log_prob(w)
        if accumulate:
            gm, gr = torch.autograd.grad(kl * weight, [mean, rho])
            self.mean.grad.add_(gm)
            self.rho.grad.add_(gr)
        return kl.detach()
