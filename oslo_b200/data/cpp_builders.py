"""ctypes front-end of the host-side index builders in ``oslo_b200/_data_C.so``."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

_LIB = None
_TRIED = False


class _Builders:
    def __init__(self, lib) -> None:
        self.lib = lib
        i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
        lib.oslo_build_sample_idx.restype = ctypes.c_int64
        lib.oslo_build_sample_idx.argtypes = [i32p, i32p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                              ctypes.c_int64, i32p, ctypes.c_int64]
        lib.oslo_build_blending_indices.restype = None
        lib.oslo_build_blending_indices.argtypes = [ctypes.POINTER(ctypes.c_uint8), i64p,
                                                    ctypes.POINTER(ctypes.c_double), ctypes.c_int32, ctypes.c_int64,
                                                    ctypes.c_void_p]
        lib.oslo_build_mapping.restype = ctypes.c_int64
        lib.oslo_build_mapping.argtypes = [i64p, ctypes.c_int64, i32p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32,
                                           ctypes.c_double, ctypes.c_int32, ctypes.c_int32, i64p, ctypes.c_int64]
        lib.oslo_build_blocks_mapping.restype = ctypes.c_int64
        lib.oslo_build_blocks_mapping.argtypes = [i64p, ctypes.c_int64, i32p, i32p, ctypes.c_int32, ctypes.c_int64,
                                                  ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, i64p, ctypes.c_int64]

    @staticmethod
    def _p(a: np.ndarray, ct):
        return a.ctypes.data_as(ctypes.POINTER(ct))

    def build_sample_idx(self, sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch) -> np.ndarray:
        sizes = np.ascontiguousarray(sizes, dtype=np.int32)
        doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
        rows = (int(num_epochs) * int(tokens_per_epoch) - 1) // int(seq_length) + 1
        out = np.zeros((rows, 2), dtype=np.int32)
        n = self.lib.oslo_build_sample_idx(self._p(sizes, ctypes.c_int32), self._p(doc_idx, ctypes.c_int32),
                                           len(doc_idx), int(seq_length), int(num_epochs), int(tokens_per_epoch),
                                           self._p(out, ctypes.c_int32), rows)
        if n < 0:
            raise ValueError("build_sample_idx: inconsistent sizes / doc_idx / tokens_per_epoch")
        return out

    def build_blending_indices(self, dataset_index, dataset_sample_index, weights, num_datasets, size, verbose=False):
        weights = np.ascontiguousarray(weights, dtype=np.float64)
        assert dataset_index.dtype == np.uint8 and dataset_sample_index.dtype == np.int64
        self.lib.oslo_build_blending_indices(self._p(dataset_index, ctypes.c_uint8),
                                             self._p(dataset_sample_index, ctypes.c_int64),
                                             self._p(weights, ctypes.c_double), int(num_datasets), int(size), None)

    def build_mapping(self, docs, sizes, num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed,
                      verbose=False, min_num_sent=2) -> np.ndarray:
        docs = np.ascontiguousarray(docs, dtype=np.int64)
        sizes = np.ascontiguousarray(sizes, dtype=np.int32)
        args = (self._p(docs, ctypes.c_int64), len(docs), self._p(sizes, ctypes.c_int32), int(num_epochs),
                int(max_num_samples), int(max_seq_length), float(short_seq_prob), int(seed), int(min_num_sent))
        n = self.lib.oslo_build_mapping(*args, None, 0)
        out = np.zeros((n, 3), dtype=np.int64)
        if n:
            self.lib.oslo_build_mapping(*args, self._p(out, ctypes.c_int64), n)
        return out

    def build_blocks_mapping(self, docs, sizes, titles_sizes, num_epochs, max_num_samples, max_seq_length, seed,
                             verbose=False, use_one_sent_blocks=False) -> np.ndarray:
        docs = np.ascontiguousarray(docs, dtype=np.int64)
        sizes = np.ascontiguousarray(sizes, dtype=np.int32)
        titles = np.ascontiguousarray(titles_sizes, dtype=np.int32)
        args = (self._p(docs, ctypes.c_int64), len(docs), self._p(sizes, ctypes.c_int32), self._p(titles, ctypes.c_int32),
                int(num_epochs), int(max_num_samples), int(max_seq_length), int(seed), int(bool(use_one_sent_blocks)))
        n = self.lib.oslo_build_blocks_mapping(*args, None, 0)
        out = np.zeros((n, 4), dtype=np.int64)
        if n:
            self.lib.oslo_build_blocks_mapping(*args, self._p(out, ctypes.c_int64), n)
        return out


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_data_C.so")


def load() -> Optional[_Builders]:
    """The builders object, or ``None`` when the library has not been built (callers fall back to NumPy)."""
    global _LIB, _TRIED
    if not _TRIED:
        _TRIED = True
        try:
            _LIB = _Builders(ctypes.CDLL(lib_path()))
        except OSError:
            _LIB = None
    return _LIB
