"""Epoch iterators over pre-cut batches.

``DataIterator`` owns the list of batches of a ``Dataset``; every epoch it shuffles the batch order with
``seed + epoch``, splits it evenly across ranks (ranks that would come up short are topped up with randomly
re-drawn batches so that all ranks take the same number of steps, which collective-based training needs),
and serves the shard of this rank through a ``torch.utils.data.DataLoader`` (worker processes collate and
pack on the host) with optional background buffering and pinned memory.  The position inside an epoch is
part of ``state_dict`` so training can resume mid-epoch.  ``MultiDataIterator`` round-robins over several
datasets in proportion to their sizes.

Reference behaviour: onmt/data/data_iterator.py:129-301 (``DataIterator``), :304-353 (``ShardedIterator``),
:356-434 (buffered iterator); onmt/data/multidata_iterator.py:15-120.
"""
from __future__ import annotations

import queue
import threading
from typing import List, Optional

import numpy as np
import torch


class _BatchIndexDataset(torch.utils.data.Dataset):
    def __init__(self, dataset, order: List[int]):
        self.dataset, self.order = dataset, order

    def __len__(self):
        return len(self.order)

    def __getitem__(self, i):
        return self.dataset.get_batch(self.order[i])


class CountingIterator:
    """Wraps an iterable, counts consumed items, and can skip a prefix (for resuming)."""

    def __init__(self, iterable, total: int, start: int = 0):
        self.iterable, self.total, self.count = iterable, total, start
        self._it = iter(iterable)

    def __len__(self):
        return self.total

    def __iter__(self):
        return self

    def __next__(self):
        item = next(self._it)
        self.count += 1
        return item

    def has_next(self):
        return self.count < self.total


class BufferedIterator:
    """Producer thread that keeps up to ``size`` ready batches; worker exceptions surface in the consumer."""

    _END = object()

    def __init__(self, iterable, size: int):
        self.q: "queue.Queue" = queue.Queue(maxsize=max(1, size))
        self.iterable = iterable
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        try:
            for item in self.iterable:
                self.q.put(item)
            self.q.put(self._END)
        except BaseException as exc:  # noqa: BLE001 - forwarded
            self.q.put(exc)

    def __iter__(self):
        return self

    def __next__(self):
        item = self.q.get()
        if item is self._END:
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        return item


def shard_order(order: List[int], num_shards: int, shard_id: int, split_even: bool, rng: np.random.RandomState) -> List[int]:
    """Strided shard of ``order``; with ``split_even`` every shard gets ceil(n / shards) items."""
    shard = order[shard_id::num_shards]
    if split_even and num_shards > 1:
        want = (len(order) + num_shards - 1) // num_shards
        while len(shard) < want and order:
            shard.append(order[int(rng.randint(0, len(order)))])
    return shard


class DataIterator:
    def __init__(self, dataset, seed: int = 1, num_workers: int = 0, epoch: float = 1.0, buffer_size: int = 0,
                 num_shards: int = 1, shard_id: int = 0, split_even: bool = True, pin_memory: bool = False,
                 shuffle: bool = True):
        self.dataset = dataset
        self.seed, self.num_workers, self.buffer_size = seed, num_workers, buffer_size
        self.num_shards, self.shard_id, self.split_even = num_shards, shard_id, split_even
        self.pin_memory, self.shuffle = pin_memory, shuffle
        self.epoch = int(epoch)
        self._resume_offset = 0
        self._cur: Optional[CountingIterator] = None

    def __len__(self):
        n = len(self.dataset)
        return (n + self.num_shards - 1) // self.num_shards if self.split_even else len(range(self.shard_id, n, self.num_shards))

    def _order_for_epoch(self, epoch: int) -> List[int]:
        order = list(range(len(self.dataset)))
        rng = np.random.RandomState(self.seed + epoch)
        if self.shuffle:
            rng.shuffle(order)
        return shard_order(order, self.num_shards, self.shard_id, self.split_even, rng)

    def next_epoch_itr(self, shuffle: Optional[bool] = None, pin_memory: Optional[bool] = None) -> CountingIterator:
        if shuffle is not None:
            self.shuffle = shuffle
        if pin_memory is not None:
            self.pin_memory = pin_memory
        order = self._order_for_epoch(self.epoch)
        start = min(self._resume_offset, len(order))
        self._resume_offset = 0
        ds = _BatchIndexDataset(self.dataset, order[start:])
        pin = self.pin_memory and torch.cuda.is_available()
        # a generator of its own: the loader draws its base seed when iteration starts, and taking that draw from the
        # global generator would shift every later dropout mask (a resumed run creates the loader at a different point
        # of the random stream than the run it continues)
        gen = torch.Generator()
        gen.manual_seed(int(self.seed) * 1000003 + int(self.epoch))
        loader = torch.utils.data.DataLoader(ds, batch_size=None, shuffle=False, num_workers=self.num_workers,
                                             collate_fn=None, pin_memory=False, generator=gen)
        it = (b.pin_memory() if pin else b for b in loader)
        if self.buffer_size > 0:
            it = BufferedIterator(it, self.buffer_size)
        self._cur = CountingIterator(it, len(order), start)
        self.epoch += 1
        return self._cur

    def end_of_epoch(self) -> bool:
        return self._cur is None or not self._cur.has_next()

    @property
    def iterations_in_epoch(self) -> int:
        return self._cur.count if self._cur is not None else 0

    def state_dict(self):
        epoch = self.epoch - 1 if (self._cur is not None and self._cur.has_next()) else self.epoch
        return {"epoch": epoch, "iterations_in_epoch": self.iterations_in_epoch if not self.end_of_epoch() else 0,
                "seed": self.seed}

    def load_state_dict(self, sd):
        self.epoch = int(sd.get("epoch", self.epoch))
        self._resume_offset = int(sd.get("iterations_in_epoch", 0))
        self.seed = sd.get("seed", self.seed)


class MultiDataIterator:
    """Interleaves several ``DataIterator`` objects; dataset i is drawn with probability ~ its length, so an epoch is
    one pass over all of them.  With ``probabilities`` (e.g. equal weights) the source of every batch is drawn with
    those weights and the epoch ends when the first data set runs out, with a schedule that changes every epoch
    (reference: whisper/trainers/trainer_shuffle_ctc.py:231-239, equal-probability interleaving reseeded per call)."""

    def __init__(self, datasets, seed: int = 1, dataset_ids=None, probabilities=None, **kw):
        self.probabilities = None if probabilities is None else [float(p) / sum(probabilities) for p in probabilities]
        ids = list(range(len(datasets))) if dataset_ids is None else list(dataset_ids)
        self.iterators = [DataIterator(datasets[i], seed=seed + 17 * i, **kw) for i in ids]
        self.seed = seed
        self.epoch = int(kw.get("epoch", 1))
        self._active = None
        self._schedule: List[int] = []
        self._pos = 0

    def __len__(self):
        return len(self._schedule) if (self.probabilities is not None and self._schedule) else sum(len(it) for it in self.iterators)

    def next_epoch_itr(self, **kw):
        self._active = [it.next_epoch_itr(**kw) for it in self.iterators]
        rng = np.random.RandomState(self.seed + self.epoch)
        if self.probabilities is None:
            sched = [i for i, it in enumerate(self.iterators) for _ in range(len(it))]
            rng.shuffle(sched)
        else:
            left = [len(it) for it in self.iterators]
            sched = []
            for i in rng.choice(len(left), size=sum(left), p=self.probabilities).tolist():
                if left[i] == 0:
                    break               # first data set exhausted: the epoch ends here
                left[i] -= 1
                sched.append(i)
        self._schedule, self._pos = sched, 0
        self.epoch += 1
        return self

    def __iter__(self):
        return self

    def __next__(self):
        if self._pos >= len(self._schedule):
            raise StopIteration
        i = self._schedule[self._pos]
        self._pos += 1
        return next(self._active[i])

    def end_of_epoch(self):
        return self._pos >= len(self._schedule)

    def state_dict(self):
        return {"epoch": self.epoch, "pos": self._pos, "iters": [it.state_dict() for it in self.iterators]}

    def load_state_dict(self, sd):
        self.epoch = sd.get("epoch", self.epoch)
        for it, s in zip(self.iterators, sd.get("iters", [])):
            it.load_state_dict(s)
