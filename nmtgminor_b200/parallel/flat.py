"""Flat parameter / gradient storage.

All trainable parameters of a model are re-homed into ONE fp32 master buffer; a bf16 working copy and an
fp32 gradient buffer have the same layout.  Each ``nn.Parameter`` becomes a view of the master buffer and
gains two attributes, ``work`` (bf16 view used by the fused kernels) and ``main_grad`` (fp32 view the
kernels accumulate weight gradients into).  With this layout

* the optimiser is a single grid-stride kernel over the flat buffers (no multi-tensor chunk tables),
* data-parallel gradient reduction works on contiguous buckets without packing copies, and
* the buffers can be placed in peer-mapped (symmetric) memory so that other GPUs read them directly.

The reference keeps per-tensor fp32 parameters under autocast and lets DistributedDataParallel build its
own 25 MB buckets (onmt/train_utils/mp_trainer.py:381-387); its flattened-parameter mode lives in
onmt/optim.py:336-386.
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Optional

import torch

ALIGN = 64  # elements; keeps every view 128-byte (bf16) / 256-byte (fp32) aligned


def _unique_params(params: Iterable[torch.nn.Parameter]) -> List[torch.nn.Parameter]:
    seen, out = set(), []
    for p in params:
        if id(p) not in seen:
            seen.add(id(p))
            out.append(p)
    return out


class FlatParameterStore:
    """Owns the flat master / working / gradient buffers of a model."""

    def __init__(self, module: torch.nn.Module, device=None, work_dtype=torch.bfloat16,
                 allocator=None,   # callable(numel, dtype) -> tensor, or {'master' | 'grad' | 'work': callable}
                 pad_total_to: int = ALIGN):
        params = _unique_params(p for p in module.parameters())
        # trainable parameters first: the optimiser (and its state) then covers one contiguous prefix of the flat space,
        # which is what makes adapter fine-tuning (a few trainable matrices in a frozen model) cheap
        params = [p for p in params if p.requires_grad] + [p for p in params if not p.requires_grad]
        self.params = params
        self.device = torch.device(device) if device is not None else (params[0].device if params else torch.device("cpu"))
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.total = (off + pad_total_to - 1) // pad_total_to * pad_total_to if off else 0
        n_train = 0
        for p, o in zip(params, self.offsets):
            if p.requires_grad:
                n_train = o + (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        # length of the trainable prefix (whole buffer when nothing is frozen, so padding stays included)
        self.trainable_total = self.total if all(p.requires_grad for p in params) else n_train
        default = lambda n, dt: torch.zeros(n, dtype=dt, device=self.device)
        allocs = allocator if isinstance(allocator, dict) else {"master": allocator, "grad": allocator, "work": allocator}
        pick = lambda name: allocs.get(name) or default
        self.master = pick("master")(self.total, torch.float32)
        self.grad = pick("grad")(self.total, torch.float32)
        self.work = pick("work")(self.total, work_dtype) if self.device.type == "cuda" else None
        self.trainable_mask = None
        for p, o in zip(params, self.offsets):
            n = p.numel()
            view = self.master[o:o + n].view(p.shape)
            with torch.no_grad():
                view.copy_(p.data.to(self.device, torch.float32))
            p.data = view
            if self.grad is not None:
                p.main_grad = self.grad[o:o + n].view(p.shape)
            if self.work is not None:
                p.work = self.work[o:o + n].view(p.shape)
        # buffers that enter the fused kernels as bf16 operands get a working copy too
        self.sync_work()
        frozen = [(o, p.numel()) for p, o in zip(params, self.offsets) if not p.requires_grad]
        self.frozen_ranges = frozen

    # ------------------------------------------------------------------------------------------
    def sync_work(self) -> None:
        """Refresh the bf16 working copy from the fp32 master (after loading a checkpoint)."""
        if self.work is None:
            return
        from .. import ops
        if ops.extension_available() and self.total % 4 == 0:
            ops.ext().cast_f32_bf16(self.master, self.work)
        else:
            self.work.copy_(self.master)

    def zero_grad(self) -> None:
        if self.grad is not None:
            self.grad.zero_()
        else:     # gradients live in buffers owned by the fully sharded step
            for p in self.params:
                g = getattr(p, "main_grad", None)
                if g is not None:
                    g.zero_()

    def gather_autograd_grads(self) -> None:
        """Add ``p.grad`` tensors (from unfused / CPU ops) into the flat gradient buffer and drop them."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    def zero_frozen_grads(self) -> None:
        if self.grad is None:
            return
        for o, n in self.frozen_ranges:
            self.grad[o:o + n].zero_()

    def named_views(self, module: torch.nn.Module):
        ids = {id(p): i for i, p in enumerate(self.params)}
        for name, p in module.named_parameters():
            i = ids[id(p)]
            yield name, self.offsets[i], p.numel()
