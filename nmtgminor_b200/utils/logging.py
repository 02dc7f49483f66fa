"""Rank-aware console logger and simple meters.

The reference prints from rank 0 (onmt/train_utils/mp_trainer.py:425-436) and ships unused ``Logger`` /
``AverageMeter`` helpers (onmt/train_utils/stats.py:10, meters.py:11-56); these are their working
counterparts.
"""
from __future__ import annotations

import sys
import time


class Logger:
    def __init__(self, enabled: bool = True, stream=None):
        self.enabled = enabled
        self.stream = stream or sys.stdout

    def __call__(self, *args, **kw):
        if self.enabled:
            print(*args, file=self.stream, flush=True, **kw)


class AverageMeter:
    def __init__(self):
        self.reset()

    def reset(self):
        self.val = self.sum = self.count = 0.0

    def update(self, val, n=1):
        self.val = val
        self.sum += val * n
        self.count += n

    @property
    def avg(self):
        return self.sum / self.count if self.count else 0.0


class TimeMeter:
    def __init__(self):
        self.reset()

    def reset(self):
        self.start, self.n = time.time(), 0.0

    def update(self, n=1):
        self.n += n

    @property
    def rate(self):
        return self.n / max(time.time() - self.start, 1e-9)


class StopwatchMeter:
    def __init__(self):
        self.sum, self.n, self._t = 0.0, 0, None

    def start(self):
        self._t = time.time()

    def stop(self, n=1):
        if self._t is not None:
            self.sum += time.time() - self._t
            self.n += n
            self._t = None

    @property
    def avg(self):
        return self.sum / self.n if self.n else 0.0
