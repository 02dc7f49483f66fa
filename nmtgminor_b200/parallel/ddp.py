"""Data-parallel gradient reduction over the flat gradient buffer.

Two reducers share one interface (``reducer(flat_grad)`` enqueues work on the current stream):

* ``nccl``  - ``torch.distributed.all_reduce`` on the flat fp32 buffer (the baseline path; also what the CPU
  tests run with the gloo backend);
* ``fused`` - the peer-memory kernels of ``parallel/symmetric.py`` (per-layer reduce-scatter by direct loads
  from every peer's gradient buffer, overlapped with the backward pass and followed by the Adam(W) update of
  the owned pieces and the write-back of the updated parameters to every peer); ``train.engine.TrainEngine``
  builds it when the symmetric heap can be set up.

Gradients are summed, not averaged: the reference trains on token-summed losses and normalises (or not)
with ``-normalize_gradient`` afterwards (onmt/train_utils/mp_trainer.py:965-979).  The reference itself relies
on ``DistributedDataParallel`` buckets (mp_trainer.py:381-387) and has a manual 10 MB bucket helper
(``all_reduce_and_rescale_tensors``, mp_trainer.py:98-149).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def broadcast_parameters(store, src: int = 0) -> None:
    """Make every rank start from rank ``src``'s master weights, then refresh the bf16 working copies."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(store.master, src)
        store.sync_work()


class NcclReducer:
    def __init__(self, world_size: int, bucket_bytes: int = 0):
        self.world_size = world_size
        self.bucket_elems = bucket_bytes // 4

    def __call__(self, flat_grad: torch.Tensor) -> None:
        if self.world_size <= 1:
            return
        if self.bucket_elems <= 0 or flat_grad.numel() <= self.bucket_elems:
            dist.all_reduce(flat_grad)
            return
        for off in range(0, flat_grad.numel(), self.bucket_elems):
            dist.all_reduce(flat_grad[off:off + self.bucket_elems])
