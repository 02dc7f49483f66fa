"""Memory-mapped indexed datasets in the fairseq ``MMIDIDX`` layout (interchangeable with the reference's
files, onmt/data/mmap_indexed_dataset.py:53-232) and the older "TNTIDX" indexed format
(onmt/data/indexed_dataset.py:51-155).

``<prefix>.idx``:  magic ``MMIDIDX\\0\\0`` | version u64 = 1 | dtype code u8 | count u64 | sizes int32[count] |
                   pointers int64[count];   ``<prefix>.bin``: the concatenated arrays.
Reading maps both files; ``dataset[i]`` is a zero-copy torch view converted to int64 on access.
"""
from __future__ import annotations

import os
import struct
from typing import Iterable

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


def index_path(prefix: str) -> str:
    return prefix + ".idx"


def data_path(prefix: str) -> str:
    return prefix + ".bin"


def best_dtype(vocab_size: int):
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


class MMapIndexedDatasetBuilder:
    def __init__(self, prefix: str, dtype=np.int32):
        self.prefix = prefix
        self.dtype = np.dtype(dtype)
        self._bin = open(data_path(prefix), "wb")
        self._sizes = []

    def add_item(self, tensor) -> None:
        arr = np.asarray(tensor.numpy() if isinstance(tensor, torch.Tensor) else tensor, dtype=self.dtype)
        self._bin.write(arr.tobytes(order="C"))
        self._sizes.append(arr.size)

    def merge_file(self, other_prefix: str) -> None:
        other = MMapIndexedDataset(other_prefix)
        assert other.dtype == self.dtype
        self._sizes.extend(int(s) for s in other.sizes)
        with open(data_path(other_prefix), "rb") as fh:
            while True:
                chunk = fh.read(1 << 24)
                if not chunk:
                    break
                self._bin.write(chunk)

    def finalize(self) -> None:
        self._bin.close()
        sizes = np.asarray(self._sizes, dtype=np.int32)
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        with open(index_path(self.prefix), "wb") as fh:
            fh.write(_MAGIC)
            fh.write(struct.pack("<Q", 1))
            fh.write(struct.pack("<B", _CODES[self.dtype]))
            fh.write(struct.pack("<Q", len(sizes)))
            fh.write(sizes.tobytes(order="C"))
            fh.write(pointers.tobytes(order="C"))


class MMapIndexedDataset(torch.utils.data.Dataset):
    def __init__(self, prefix: str):
        self.prefix = prefix
        with open(index_path(prefix), "rb") as fh:
            magic = fh.read(9)
            if magic != _MAGIC:
                raise ValueError("%s is not an MMIDIDX index file" % index_path(prefix))
            (version,) = struct.unpack("<Q", fh.read(8))
            if version != 1:
                raise ValueError("unsupported index version %d" % version)
            (code,) = struct.unpack("<B", fh.read(1))
            self.dtype = np.dtype(_DTYPES[code])
            (self._len,) = struct.unpack("<Q", fh.read(8))
            offset = fh.tell()
        self._index = np.memmap(index_path(prefix), mode="r", order="C")
        self.sizes = np.frombuffer(self._index, dtype=np.int32, count=self._len, offset=offset)
        self._pointers = np.frombuffer(self._index, dtype=np.int64, count=self._len, offset=offset + self.sizes.nbytes)
        self._data = np.memmap(data_path(prefix), mode="r", order="C") if self._len else None

    def __len__(self):
        return self._len

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(self._len))]
        if i < 0:
            i += self._len
        arr = np.frombuffer(self._data, dtype=self.dtype, count=int(self.sizes[i]), offset=int(self._pointers[i]))
        if self.dtype in (np.float32, np.float64):
            return torch.from_numpy(arr.astype(np.float32))
        return torch.from_numpy(arr.astype(np.int64))

    @staticmethod
    def exists(prefix: str) -> bool:
        return os.path.exists(index_path(prefix)) and os.path.exists(data_path(prefix))


def write_dataset(prefix: str, items: Iterable, dtype=np.int32) -> None:
    b = MMapIndexedDatasetBuilder(prefix, dtype)
    for it in items:
        b.add_item(it)
    b.finalize()


# ---------------------------------------------------------------------------------------------------
# legacy "TNTIDX" format: header | code | element size | count | total | dim_offsets | data_offsets | sizes
# ---------------------------------------------------------------------------------------------------
class IndexedDataset(torch.utils.data.Dataset):
    _HDR = b"TNTIDX\x00\x00"

    def __init__(self, prefix: str):
        with open(index_path(prefix), "rb") as fh:
            if fh.read(8) != self._HDR:
                raise ValueError("not a TNTIDX index file")
            (version,) = struct.unpack("<Q", fh.read(8))
            code, self.element_size = struct.unpack("<QQ", fh.read(16))
            self.dtype = np.dtype(_DTYPES[code])
            self._len, s = struct.unpack("<QQ", fh.read(16))
            self.dim_offsets = np.fromfile(fh, dtype=np.int64, count=self._len + 1)
            self.data_offsets = np.fromfile(fh, dtype=np.int64, count=self._len + 1)
            self.sizes = np.fromfile(fh, dtype=np.int64, count=s)
        self._data = np.memmap(data_path(prefix), mode="r", order="C")

    def __len__(self):
        return self._len

    def __getitem__(self, i):
        shape = tuple(int(x) for x in self.sizes[self.dim_offsets[i]:self.dim_offsets[i + 1]])
        n = int(np.prod(shape))
        arr = np.frombuffer(self._data, dtype=self.dtype, count=n, offset=int(self.data_offsets[i]) * self.element_size)
        t = torch.from_numpy(arr.reshape(shape).copy())
        return t.long() if not t.is_floating_point() else t


class IndexedDatasetBuilder:
    def __init__(self, prefix: str, dtype=np.int32):
        self.prefix, self.dtype = prefix, np.dtype(dtype)
        self._bin = open(data_path(prefix), "wb")
        self.data_offsets, self.dim_offsets, self.sizes = [0], [0], []

    def add_item(self, tensor):
        arr = np.asarray(tensor.numpy() if isinstance(tensor, torch.Tensor) else tensor, dtype=self.dtype)
        self._bin.write(arr.tobytes(order="C"))
        self.data_offsets.append(self.data_offsets[-1] + arr.size)
        self.sizes.extend(arr.shape)
        self.dim_offsets.append(self.dim_offsets[-1] + arr.ndim)

    def finalize(self):
        self._bin.close()
        with open(index_path(self.prefix), "wb") as fh:
            fh.write(IndexedDataset._HDR)
            fh.write(struct.pack("<Q", 1))
            fh.write(struct.pack("<QQ", _CODES[self.dtype], self.dtype.itemsize))
            fh.write(struct.pack("<QQ", len(self.data_offsets) - 1, len(self.sizes)))
            np.asarray(self.dim_offsets, dtype=np.int64).tofile(fh)
            np.asarray(self.data_offsets, dtype=np.int64).tofile(fh)
            np.asarray(self.sizes, dtype=np.int64).tofile(fh)
