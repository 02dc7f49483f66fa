"""Dynamic loss scaling with the scale resident on the device.

The loss gradient is multiplied by ``scale`` where it is born (the fused cross-entropy reads the 1-element device tensor
``scaler.scale``), the optimiser's gradient factor is divided by it on the device right before the update kernels
(``prepare``), and after them ``update`` looks at the step's non-finite flag: a skipped step halves the scale, ``interval``
clean steps in a row double it.  Nothing is read back by the host, so the protocol is part of a captured CUDA graph and
costs two one-thread kernels per step.  On the CPU the same arithmetic runs as tensor ops (tests, gloo runs).

The update kernels themselves already skip on a non-finite gradient - on every rank, because the sharded update exchanges
the flag with the norm - so parameters and moments are untouched by an overflowing step.

``state_dict()`` / ``load_state_dict()`` are what the trainer stores under the checkpoint key ``'scaler'`` (the key the
reference uses for its ``GradScaler`` state).

Reference: onmt/train_utils/mp_trainer.py:294-312 (``GradScaler`` creation), :970 (``scale(loss).backward()``),
:1015-1016 (``step`` / ``update``); torch.cuda.amp.GradScaler for the growth / back-off rule.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch


class DynamicLossScaler:
    def __init__(self, device, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, min_scale: float = 1.0, max_scale: float = 2.0 ** 24):
        self.device = torch.device(device)
        self.growth_factor, self.backoff_factor = float(growth_factor), float(backoff_factor)
        self.growth_interval = int(growth_interval)
        self.min_scale, self.max_scale = float(min_scale), float(max_scale)
        # { scale, clean steps since the last change, 1 / scale, skipped steps }
        self.state = torch.tensor([init_scale, 0.0, 1.0 / init_scale, 0.0], dtype=torch.float32, device=self.device)

    @property
    def scale(self) -> torch.Tensor:
        """1-element view handed to the loss as ``grad_scale``."""
        return self.state[0:1]

    def prepare(self, hyper: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Folds ``1 / scale`` into the optimiser's device-side gradient factor (``hyper`` is the optimiser's parameter
        block).  Without a block (unfused optimisers) returns the ``1 / scale`` tensor for the caller to multiply by."""
        if hyper is None:
            return self.state[2:3]
        if hyper.is_cuda:
            from .. import ops
            ops.ext().loss_scale_prepare(hyper, self.state)
        else:
            hyper[7] = hyper[7] / self.state[0]
        return None

    def update(self, nonfinite: Optional[torch.Tensor] = None, norm: Optional[torch.Tensor] = None) -> None:
        """``nonfinite``: int32 flag of the local update; ``norm``: global gradient norm of the sharded update, negative
        when the step was skipped.  Either may be missing."""
        if self.state.is_cuda:
            from .. import ops
            ops.ext().loss_scale_update(self.state, nonfinite, norm, self.growth_interval, self.growth_factor,
                                        self.backoff_factor, self.min_scale, self.max_scale)
            return
        skipped = torch.zeros((), dtype=torch.bool)
        if nonfinite is not None:
            skipped = skipped | (nonfinite.reshape(-1)[0] != 0)
        if norm is not None:
            skipped = skipped | ~(norm.reshape(-1)[0] >= 0)
        s, clean = self.state[0], self.state[1]
        if bool(skipped):
            s = torch.clamp(s * self.backoff_factor, min=self.min_scale)
            clean = torch.zeros(())
            self.state[3] += 1
        else:
            clean = clean + 1
            if float(clean) >= self.growth_interval:
                s = torch.clamp(s * self.growth_factor, max=self.max_scale)
                clean = torch.zeros(())
        self.state[0], self.state[1], self.state[2] = s, clean, 1.0 / s

    # host-side views (each of these synchronises: for logging and checkpoints only)
    def get_scale(self) -> float:
        return float(self.state[0])

    def skipped_steps(self) -> int:
        return int(self.state[3])

    def state_dict(self) -> Dict:
        s = self.state.detach().cpu().tolist()
        return {"scale": s[0], "growth_tracker": int(s[1]), "skipped": int(s[3]), "growth_factor": self.growth_factor,
                "backoff_factor": self.backoff_factor, "growth_interval": self.growth_interval}

    def load_state_dict(self, sd: Dict) -> None:
        if not sd:
            return
        scale = float(sd.get("scale", sd.get("_scale", self.get_scale())))
        self.state.copy_(torch.tensor([scale, float(sd.get("growth_tracker", sd.get("_growth_tracker", 0))), 1.0 / scale,
                                       float(sd.get("skipped", 0))]))
        self.growth_factor = float(sd.get("growth_factor", self.growth_factor))
        self.backoff_factor = float(sd.get("backoff_factor", self.backoff_factor))
        self.growth_interval = int(sd.get("growth_interval", self.growth_interval))


def wants_loss_scaling(opt) -> bool:
    """``-fp16`` without ``-bf16`` asks for the fp16 protocol (dynamic loss scale); ``-bf16`` needs none."""
    return bool(getattr(opt, "fp16", False)) and not bool(getattr(opt, "bf16", False)) and not bool(getattr(opt, "fp32", False))
