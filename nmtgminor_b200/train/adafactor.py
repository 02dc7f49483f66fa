"""Adafactor (Shazeer & Stern 2018): factored second moments, relative step sizes, update clipping.

Counterpart of the reference's ``Adafactor`` class (onmt/optim.py:29-228).  The second moment of a matrix is kept
as a row vector and a column vector; ``lr=None`` enables the relative step ``min(1e-2, 1/sqrt(t))`` scaled by
the parameter RMS.
"""
from __future__ import annotations

import math

import torch


class Adafactor(torch.optim.Optimizer):
    def __init__(self, params, lr=None, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8, beta1=None, weight_decay=0.0,
                 scale_parameter=True, relative_step=None, warmup_init=False):
        relative_step = (lr is None) if relative_step is None else relative_step
        defaults = dict(lr=lr, eps=eps, clip_threshold=clip_threshold, decay_rate=decay_rate, beta1=beta1,
                        weight_decay=weight_decay, scale_parameter=scale_parameter, relative_step=relative_step,
                        warmup_init=warmup_init)
        super().__init__(params, defaults)

    @staticmethod
    def _rms(t):
        return t.norm(2) / (t.numel() ** 0.5)

    def _lr(self, group, state):
        lr = group["lr"]
        if group["relative_step"]:
            min_step = 1e-6 * state["step"] if group["warmup_init"] else 1e-2
            lr = min(min_step, 1.0 / math.sqrt(state["step"]))
        scale = max(group["eps"][1], state["RMS"]) if group["scale_parameter"] else 1.0
        return scale * lr

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                state = self.state[p]
                factored = g.dim() >= 2
                if not state:
                    state["step"] = 0
                    if group["beta1"] is not None:
                        state["exp_avg"] = torch.zeros_like(g)
                    if factored:
                        state["row"] = torch.zeros(g.shape[:-1], dtype=torch.float32, device=g.device)
                        state["col"] = torch.zeros(g.shape[:-2] + g.shape[-1:], dtype=torch.float32, device=g.device)
                    else:
                        state["sq"] = torch.zeros_like(g)
                    state["RMS"] = 0.0
                state["step"] += 1
                pf = p.data.float()
                state["RMS"] = float(self._rms(pf))
                lr = self._lr(group, state)
                beta2 = 1.0 - state["step"] ** group["decay_rate"]
                upd = g * g + group["eps"][0]
                if factored:
                    state["row"].mul_(beta2).add_(upd.mean(-1), alpha=1 - beta2)
                    state["col"].mul_(beta2).add_(upd.mean(-2), alpha=1 - beta2)
                    r = (state["row"] / state["row"].mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
                    c = state["col"].rsqrt().unsqueeze(-2)
                    upd = g * r * c
                else:
                    state["sq"].mul_(beta2).add_(upd, alpha=1 - beta2)
                    upd = g * state["sq"].rsqrt()
                upd.div_(max(1.0, float(self._rms(upd)) / group["clip_threshold"]))
                upd.mul_(lr)
                if group["beta1"] is not None:
                    state["exp_avg"].mul_(group["beta1"]).add_(upd, alpha=1 - group["beta1"])
                    upd = state["exp_avg"]
                if group["weight_decay"]:
                    pf.add_(pf, alpha=-group["weight_decay"] * lr)
                pf.add_(-upd)
                p.data.copy_(pf)
        return loss
