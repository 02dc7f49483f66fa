"""Host-side failure detection for multi-process training.

Every rank runs a ``Heartbeat``: a daemon thread that publishes ``(update count, wall time)`` under its rank's
key in a key-value store (``torch.distributed.TCPStore``, or any object with ``set`` / ``get``) and checks the
other ranks' keys.  A rank whose heartbeat is older than ``timeout`` seconds is reported through
``on_failure`` (default: raise ``RankFailure`` in the training thread at its next ``beat``), so the job stops
between steps, with no kernel or collective of the survivor in flight, instead of waiting inside a
collective for a peer that is gone.  Device-side waits have their own bound (the fused kernels give up after
a fixed number of polls and set the status word that the trainer checks); this module covers everything the
host can see earlier: a crashed or wedged process, a data loader that stopped producing.

The reference has no failure detection (NCCL default timeouts only; onmt/train_utils/mp_trainer.py:914-950
catches OOM to print shapes and re-raises).
"""
from __future__ import annotations

import json
import threading
import time
from typing import Callable, Dict, Optional


class RankFailure(RuntimeError):
    pass


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process runs)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k, v):
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        with self._lock:
            if k not in self._d:
                raise KeyError(k)
            return self._d[k]

    def check(self, keys):
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    def __init__(self, rank: int, world_size: int, timeout: float = 60.0, interval: Optional[float] = None, store=None,
                 on_failure: Optional[Callable[[int, float], None]] = None, clock: Callable[[], float] = time.time,
                 start: bool = True):
        self.rank, self.world, self.timeout = rank, world_size, timeout
        self.interval = interval if interval is not None else max(0.05, timeout / 4.0)
        self.store = store if store is not None else self._default_store()
        self.on_failure = on_failure
        self.clock = clock
        self.step = 0
        self.failed: Optional[int] = None
        self._stop = threading.Event()
        self._t0 = clock()
        self._publish()
        self.thread = threading.Thread(target=self._loop, daemon=True)
        if start:
            self.thread.start()

    def _default_store(self):
        import os
        import torch.distributed as dist
        host = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("MASTER_PORT", "29500")) + 17
        return dist.TCPStore(host, port, self.world, is_master=(self.rank == 0), wait_for_workers=False)

    def _publish(self):
        self.store.set("hb/%d" % self.rank, json.dumps({"step": self.step, "time": self.clock()}).encode())

    def check_peers(self) -> Optional[int]:
        """Returns the rank of a peer whose heartbeat is stale (or was never seen within the timeout)."""
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                rec = json.loads(bytes(self.store.get("hb/%d" % r)).decode())
                age = now - rec["time"]
            except Exception:  # noqa: BLE001 - missing key: count from start-up
                age = now - self._t0
            if age > self.timeout:
                return r
        return None

    def _loop(self):
        while not self._stop.wait(self.interval):
            try:
                self._publish()
                bad = self.check_peers()
            except Exception:  # noqa: BLE001 - the store itself went away: treat the master as failed
                bad = 0 if self.rank != 0 else None
            if bad is not None and self.failed is None:
                self.failed = bad
                if self.on_failure is not None:
                    self.on_failure(bad, self.timeout)

    def beat(self, step: int):
        """Called by the training loop between steps; raises when a peer was found dead."""
        self.step = step
        if self.failed is not None:
            raise RankFailure("rank %d sent no heartbeat for more than %.1f s" % (self.failed, self.timeout))

    def stop(self):
        self._stop.set()
