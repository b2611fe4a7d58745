"""On-disk token stores: ``<name>.bin`` (raw tokens) + ``<name>.idx`` (sizes / pointers / document index).

Three readers over two index formats, byte-compatible with the reference
(oslo/data/indexing/mmap_indexing.py:272-463, lazy_indexing.py:83-250, cached_indexing.py:16-126):

* ``mmap``   - magic ``MMIDIDX\\0\\0``, u64 version 1, u8 dtype code, u64 #sizes, u64 #docs, i32 sizes,
               i64 byte pointers, i64 document index; data is memory-mapped.
* ``lazy``   - magic ``TNTIDX\\0\\0``, u64 version, (u64 dtype code, u64 element size), (u64 #items, u64 #sizes),
               u64 #docs, then i64 dim offsets, data offsets, sizes, document index; data read with seeks.
* ``cached`` - the lazy format with a prefetch cache.

Every reader offers ``get(idx, offset, length)`` so all three work with ``DatasetForCausalLM``.
"""
from __future__ import annotations

import os
import struct
from functools import lru_cache
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

DTYPE_BY_CODE = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64,
                 8: np.uint16}
CODE_BY_DTYPE = {np.dtype(v): k for k, v in DTYPE_BY_CODE.items()}
MMAP_MAGIC = b"MMIDIDX\x00\x00"
LAZY_MAGIC = b"TNTIDX\x00\x00"


def index_path(prefix: str) -> str:
    return prefix + ".idx"


def data_path(prefix: str) -> str:
    return prefix + ".bin"


class PathUtils:
    """``idx_path`` / ``data_path`` under the reference's class name (oslo/data/indexing/__init__.py:8-40)."""

    idx_path = staticmethod(index_path)
    data_path = staticmethod(data_path)


class NumpyUtils:
    """Dtype codes of the index formats and the two int64 array helpers of the lazy index
    (reference: oslo/data/indexing/__init__.py:43-109)."""

    dtypes_by_code = DTYPE_BY_CODE
    cody_by_dtypes = {v: k for k, v in DTYPE_BY_CODE.items()}        # (sic: the reference's spelling)
    code_by_dtypes = cody_by_dtypes
    element_sizes = {v: np.dtype(v).itemsize for v in DTYPE_BY_CODE.values()}

    @staticmethod
    def create_array_from_file(file, size) -> np.ndarray:
        """``size`` int64 values read from the binary file at its current position."""
        array = np.empty(size, dtype=np.int64)
        got = file.readinto(array)
        if got != array.nbytes:
            raise EOFError(f"wanted {array.nbytes} bytes, file had {got}")
        return array

    @staticmethod
    def write_file_from_array(file, array) -> None:
        file.write(np.asarray(array, dtype=np.int64).tobytes(order="C"))


def _as_numpy(item) -> np.ndarray:
    if isinstance(item, torch.Tensor):
        return item.detach().cpu().numpy()
    return np.asarray(item)


# ---------------------------------------------------------------------- mmap format
class MMapIndexedDatasetBuilder:
    def __init__(self, output_file_path: str, dtype=np.int32) -> None:
        self._file = open(output_file_path, "wb")
        self.dtype = np.dtype(dtype)
        self.sizes: List[int] = []
        self.doc_idx: List[int] = [0]

    def add_item(self, tensor) -> None:
        arr = np.ascontiguousarray(_as_numpy(tensor), dtype=self.dtype)
        self._file.write(arr.tobytes(order="C"))
        self.sizes.append(arr.size)

    def end_document(self) -> None:
        self.doc_idx.append(len(self.sizes))

    def merge_file_(self, another_file_path: str) -> None:
        other = MMapIndex(index_path(another_file_path))
        if other.dtype != self.dtype:
            raise ValueError("cannot merge stores of different dtypes")
        base = len(self.sizes)
        self.sizes.extend(int(s) for s in other.sizes)
        self.doc_idx.extend(int(d) + base for d in other.doc_idx[1:])
        with open(data_path(another_file_path), "rb") as f:
            while True:
                chunk = f.read(1 << 20)
                if not chunk:
                    break
                self._file.write(chunk)

    def finalize(self, index_file_path: str) -> None:
        self._file.close()
        MMapIndex.write(index_file_path, self.dtype, self.sizes, self.doc_idx)


class MMapIndex:
    """Parsed ``.idx`` of the mmap format."""

    def __init__(self, path: str) -> None:
        with open(path, "rb") as f:
            if f.read(9) != MMAP_MAGIC:
                raise ValueError(f"{path} is not an mmap index (bad magic)")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = np.dtype(DTYPE_BY_CODE[code])
            (self._len,) = struct.unpack("<Q", f.read(8))
            (self._doc_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._mmap = np.memmap(path, mode="r", order="C")
        buf = memoryview(self._mmap)
        self.sizes = np.frombuffer(buf, dtype=np.int32, count=self._len, offset=offset)
        self.pointers = np.frombuffer(buf, dtype=np.int64, count=self._len, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(buf, dtype=np.int64, count=self._doc_count,
                                     offset=offset + self.sizes.nbytes + self.pointers.nbytes)

    @staticmethod
    def write(path: str, dtype, sizes: Sequence[int], doc_idx: Sequence[int]) -> None:
        dtype = np.dtype(dtype)
        sizes_a = np.asarray(sizes, dtype=np.int32)
        pointers = np.zeros(len(sizes_a), dtype=np.int64)
        if len(sizes_a) > 1:
            np.cumsum(sizes_a[:-1].astype(np.int64) * dtype.itemsize, out=pointers[1:])
        with open(path, "wb") as f:
            f.write(MMAP_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", CODE_BY_DTYPE[dtype]))
            f.write(struct.pack("<Q", len(sizes_a)))
            f.write(struct.pack("<Q", len(doc_idx)))
            f.write(sizes_a.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(doc_idx, dtype=np.int64).tobytes(order="C"))

    def __len__(self) -> int:
        return self._len

    @lru_cache(maxsize=8)
    def __getitem__(self, i: int):
        return self.pointers[i], self.sizes[i]


MmapIndex = MMapIndex      # the reference's spelling


class MMapIndexedDataset(torch.utils.data.Dataset):
    def __init__(self, path: str) -> None:
        super().__init__()
        self._path = path
        self._open(path)

    def _open(self, path: str) -> None:
        self._index = MMapIndex(index_path(path))
        self._bin = np.memmap(data_path(path), mode="r", order="C")
        self._buf = memoryview(self._bin)

    def __getstate__(self) -> str:
        return self._path

    def __setstate__(self, state: str) -> None:
        self._path = state
        self._open(state)

    def __len__(self) -> int:
        return len(self._index)

    def __getitem__(self, idx: Union[int, slice]):
        if isinstance(idx, int):
            return self.get(idx)
        start, stop, step = idx.indices(len(self))
        if step != 1:
            raise ValueError("slices must be contiguous")
        sizes = self._index.sizes[idx]
        total = int(sizes.sum())
        flat = np.frombuffer(self._buf, dtype=self._index.dtype, count=total, offset=int(self._index.pointers[start]))
        return np.split(flat, np.cumsum(sizes)[:-1])

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        ptr, size = int(self._index.pointers[idx]), int(self._index.sizes[idx])
        if length is None:
            length = size - offset
        ptr += offset * self._index.dtype.itemsize
        return np.frombuffer(self._buf, dtype=self._index.dtype, count=length, offset=ptr)

    @property
    def dtype(self):
        """Token type of the data file."""
        return self._index.dtype

    @property
    def sizes(self) -> np.ndarray:
        return self._index.sizes

    @property
    def doc_idx(self) -> np.ndarray:
        return self._index.doc_idx

    @property
    def supports_prefetch(self) -> bool:
        return False

    @staticmethod
    def exists(path: str) -> bool:
        return os.path.exists(index_path(path)) and os.path.exists(data_path(path))

    @staticmethod
    def builder(path: str, dtype=np.int32) -> MMapIndexedDatasetBuilder:
        return MMapIndexedDatasetBuilder(path, dtype)


# ---------------------------------------------------------------------- lazy / cached format
class IndexedDatasetBuilder:
    def __init__(self, output_file_path: str, dtype=np.int32) -> None:
        self.out_file = open(output_file_path, "wb")
        self.dtype = np.dtype(dtype)
        self.element_size = self.dtype.itemsize
        self.data_offsets, self.dim_offsets, self.sizes, self.doc_idx = [0], [0], [], [0]

    def add_item(self, tensor) -> None:
        arr = np.ascontiguousarray(_as_numpy(tensor), dtype=self.dtype)
        self.out_file.write(arr.tobytes(order="C"))
        self.data_offsets.append(self.data_offsets[-1] + arr.size)
        self.sizes.extend(arr.shape)
        self.dim_offsets.append(self.dim_offsets[-1] + arr.ndim)

    def end_document(self) -> None:
        self.doc_idx.append(len(self.sizes))

    def merge_file_(self, another_file_path: str) -> None:
        other = IndexedDataset(another_file_path)
        if other.dtype != self.dtype:
            raise ValueError("cannot merge stores of different dtypes")
        base = self.data_offsets[-1]
        self.data_offsets.extend(base + int(o) for o in other.data_offsets[1:])
        self.sizes.extend(int(s) for s in other.sizes)
        base = self.dim_offsets[-1]
        self.dim_offsets.extend(base + int(o) for o in other.dim_offsets[1:])
        with open(data_path(another_file_path), "rb") as f:
            while True:
                chunk = f.read(1 << 20)
                if not chunk:
                    break
                self.out_file.write(chunk)

    def finalize(self, index_file_path: str) -> None:
        self.out_file.close()
        with open(index_file_path, "wb") as f:
            f.write(LAZY_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<QQ", CODE_BY_DTYPE[self.dtype], self.element_size))
            f.write(struct.pack("<QQ", len(self.data_offsets) - 1, len(self.sizes)))
            f.write(struct.pack("<Q", len(self.doc_idx)))
            for arr in (self.dim_offsets, self.data_offsets, self.sizes, self.doc_idx):
                f.write(np.asarray(arr, dtype=np.int64).tobytes(order="C"))


class IndexedDataset(torch.utils.data.Dataset):
    """Reads items with seek + read; nothing is kept in memory besides the index."""

    def __init__(self, path: str) -> None:
        super().__init__()
        self.path = path
        self.data_file = None
        self._read_index(path)

    def _read_index(self, path: str) -> None:
        with open(index_path(path), "rb") as f:
            if f.read(8) != LAZY_MAGIC:
                raise ValueError(f"{index_path(path)} is not a lazy index (bad magic)")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            code, self.element_size = struct.unpack("<QQ", f.read(16))
            self.dtype = np.dtype(DTYPE_BY_CODE[code])
            self._len, n_sizes = struct.unpack("<QQ", f.read(16))
            (doc_count,) = struct.unpack("<Q", f.read(8))
            rd = lambda n: np.frombuffer(f.read(8 * n), dtype=np.int64).copy()  # noqa: E731
            self.dim_offsets = rd(self._len + 1)
            self.data_offsets = rd(self._len + 1)
            self.sizes = rd(n_sizes)
            self.doc_idx = rd(doc_count)

    def read_index(self, path: str) -> None:
        """Parse ``<path>.idx`` (what the constructor does; public under the reference's name)."""
        self._read_index(path)

    def read_data(self, path: str) -> None:
        """Open ``<path>.bin`` unbuffered; otherwise it is opened at the first access."""
        if self.data_file is not None:
            self.data_file.close()
        self.data_file = open(data_path(path), "rb", buffering=0)

    def _file(self):
        if self.data_file is None:
            self.data_file = open(data_path(self.path), "rb", buffering=0)
        return self.data_file

    def __del__(self) -> None:
        if getattr(self, "data_file", None) is not None:
            self.data_file.close()

    def __getstate__(self):
        return self.path

    def __setstate__(self, state) -> None:
        self.path = state
        self.data_file = None
        self._read_index(state)

    def __len__(self) -> int:
        return self._len

    def check_index(self, i: int) -> None:
        if i < 0 or i >= self._len:
            raise IndexError("index out of range")

    def _read(self, start_elem: int, count: int) -> np.ndarray:
        out = np.empty(count, dtype=self.dtype)
        f = self._file()
        f.seek(start_elem * self.element_size)
        f.readinto(out)
        return out

    def __getitem__(self, idx: Union[int, slice]):
        if isinstance(idx, int):
            self.check_index(idx)
            shape = self.sizes[self.dim_offsets[idx]: self.dim_offsets[idx + 1]]
            return self._read(int(self.data_offsets[idx]), int(np.prod(shape))).reshape(shape)
        start, stop, step = idx.indices(len(self))
        if step != 1:
            raise ValueError("slices must be contiguous")
        flat = self._read(int(self.data_offsets[start]), int(self.data_offsets[stop] - self.data_offsets[start]))
        cuts = (self.data_offsets[start + 1: stop] - self.data_offsets[start]).astype(np.int64)
        return np.split(flat, cuts)

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        """Slice ``[offset, offset + length)`` of item ``idx`` (the reference's lazy readers lack this, which
        makes them unusable with its causal-LM dataset)."""
        self.check_index(idx)
        size = int(self.data_offsets[idx + 1] - self.data_offsets[idx])
        if length is None:
            length = size - offset
        return self._read(int(self.data_offsets[idx]) + offset, length)

    def num_tokens(self, index):
        return self.sizes[index]

    def size(self, index):
        return self.sizes[index]

    @staticmethod
    def exists(path: str) -> bool:
        return os.path.exists(index_path(path)) and os.path.exists(data_path(path))

    @property
    def supports_prefetch(self) -> bool:
        return False

    @staticmethod
    def builder(path: str, dtype=np.int32) -> IndexedDatasetBuilder:
        return IndexedDatasetBuilder(path, dtype)


class IndexedCachedDataset(IndexedDataset):
    """Lazy format with an explicit ``prefetch(indices)`` that packs the wanted items into one array."""

    def __init__(self, path: str) -> None:
        super().__init__(path)
        self.cache: Optional[np.ndarray] = None
        self.cache_index = {}

    @property
    def supports_prefetch(self) -> bool:
        return True

    def prefetch(self, indices: Sequence[int]) -> None:
        if all(i in self.cache_index for i in indices):
            return
        indices = sorted(set(int(i) for i in indices))
        total = sum(int(self.data_offsets[i + 1] - self.data_offsets[i]) for i in indices)
        self.cache = np.empty(total, dtype=self.dtype)
        self.cache_index.clear()
        ptx = 0
        for i in indices:
            n = int(self.data_offsets[i + 1] - self.data_offsets[i])
            self.cache[ptx: ptx + n] = self._read(int(self.data_offsets[i]), n)
            self.cache_index[i] = ptx
            ptx += n
        if self.data_file is not None:
            self.data_file.close()
            self.data_file = None

    def _cached(self, idx: int) -> Optional[np.ndarray]:
        if idx in self.cache_index:
            n = int(self.data_offsets[idx + 1] - self.data_offsets[idx])
            p = self.cache_index[idx]
            return self.cache[p: p + n]
        return None

    def __getitem__(self, idx):
        if isinstance(idx, int):
            hit = self._cached(idx)
            if hit is not None:
                shape = self.sizes[self.dim_offsets[idx]: self.dim_offsets[idx + 1]]
                return hit.reshape(shape).copy()
            return super().__getitem__(idx)
        return [self[i] for i in range(*idx.indices(len(self)))]

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        hit = self._cached(idx)
        if hit is None:
            return super().get(idx, offset, length)
        return hit[offset: None if length is None else offset + length].copy()


def make_builder(path: str, impl: str, dtype=np.int32):
    if impl == "mmap":
        return MMapIndexedDatasetBuilder(path, dtype)
    if impl in ("lazy", "cached"):
        return IndexedDatasetBuilder(path, dtype)
    raise ValueError(f"unknown binarization_impl {impl!r}; expected 'mmap', 'lazy' or 'cached'")


def make_dataset(path: str, impl: str):
    cls = {"mmap": MMapIndexedDataset, "lazy": IndexedDataset, "cached": IndexedCachedDataset}.get(impl)
    if cls is None:
        raise ValueError(f"unknown binarization_impl {impl!r}; expected 'mmap', 'lazy' or 'cached'")
    if not cls.exists(path):
        raise FileNotFoundError(f"{index_path(path)} / {data_path(path)} not found")
    return cls(path)
