"""Lion optimiser (sign of an interpolated momentum; Chen et al. 2023).  The reference imports it from
``lion_pytorch`` when ``-optim lion`` is chosen (onmt/optim.py:360-366); this is a self-contained version."""
from __future__ import annotations

import torch


class Lion(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p)
                m = st["exp_avg"]
                p.mul_(1 - group["lr"] * group["weight_decay"])
                upd = (m * b1 + p.grad * (1 - b1)).sign_()
                p.add_(upd, alpha=-group["lr"])
                m.mul_(b2).add_(p.grad, alpha=1 - b2)
        return loss
