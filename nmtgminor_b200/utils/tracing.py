"""NVTX ranges and device-side timing helpers.

``install_nvtx_hooks(model)`` brackets the forward pass of every layer-like module with an NVTX range named after the
module path, so an Nsight Systems / Compute timeline shows layers instead of anonymous kernels; ``nvtx_range`` is the
context manager the engine puts around forward / backward / reduction / optimiser when ``-trace_nvtx`` is set.
``CudaTimer`` measures regions with CUDA events on the current stream (never the wall clock) and reduces the maximum
over ranks; ``exposed_comm_ms`` is the usual ``step - compute_only`` estimate from two such timers.

The reference has no tracing beyond ``torch.cuda.profiler.start/stop`` brackets in its test scripts
(test/test_self_attention.py:82,102); this module is the replacement named in the build plan.
"""
from __future__ import annotations

import contextlib
from typing import Iterable, List, Optional

import torch


def _nvtx_available() -> bool:
    return torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    if enabled and _nvtx_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def install_nvtx_hooks(model: torch.nn.Module, kinds: Iterable[str] = ("Layer", "Attention", "FeedForward", "Embedding", "Generator")):
    """Returns the hook handles (call ``.remove()`` on each to uninstall)."""
    handles: List = []
    if not _nvtx_available():
        return handles
    for name, module in model.named_modules():
        if not any(k in module.__class__.__name__ for k in kinds):
            continue
        label = "%s[%s]" % (name or "model", module.__class__.__name__)
        handles.append(module.register_forward_pre_hook(lambda _m, _i, _l=label: torch.cuda.nvtx.range_push(_l)))
        handles.append(module.register_forward_hook(lambda _m, _i, _o: torch.cuda.nvtx.range_pop()))
    return handles


class CudaTimer:
    """``with timer: ...`` accumulates device time of the enclosed launches on the current stream."""

    def __init__(self):
        self.total_ms, self.count = 0.0, 0
        self._pairs = []

    def __enter__(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._start.record()
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self._pairs.append((self._start, end))
        return False

    def flush(self) -> float:
        """Synchronises once and folds the pending event pairs into ``total_ms``."""
        if self._pairs:
            torch.cuda.synchronize()
            for a, b in self._pairs:
                self.total_ms += a.elapsed_time(b)
                self.count += 1
            self._pairs = []
        return self.total_ms

    def mean_ms(self, reduce_max_over_ranks: bool = True) -> float:
        self.flush()
        v = self.total_ms / max(self.count, 1)
        if reduce_max_over_ranks and torch.distributed.is_available() and torch.distributed.is_initialized():
            t = torch.tensor([v], dtype=torch.float64, device="cuda")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            v = float(t.item())
        return v


def exposed_comm_ms(step: CudaTimer, compute_only: CudaTimer) -> float:
    return max(step.mean_ms() - compute_only.mean_ms(), 0.0)
