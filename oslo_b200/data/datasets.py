"""Packed causal-LM dataset: every sample is exactly ``max_seq_length`` tokens stitched across documents.

Three cached index arrays drive it (reference: oslo/data/datasets/dataset_causal_lm.py:163-360):
``doc_idx`` (shuffled document order), ``sample_idx[(position in doc_idx, token offset)]`` marking where
each sample starts, and ``shuffle_idx`` (sample order). They are built once by local rank 0 (C++ builder
when available, NumPy otherwise), saved as ``.npy`` beside the data and memory-mapped by everyone.
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from . import cpp_builders
from .indexing import make_dataset


def build_sample_idx_numpy(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch) -> np.ndarray:
    """NumPy statement of the sample-start table (the oracle for the C++ builder)."""
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros((num_samples + 1, 2), dtype=np.int32)
    di, offset = 0, 0
    for s in range(1, num_samples + 1):
        remaining = seq_length + 1
        while remaining != 0:
            doc_len = int(sizes[doc_idx[di]]) - offset
            remaining -= doc_len
            if remaining <= 0:
                offset += remaining + doc_len - 1
                remaining = 0
            else:
                di += 1
                offset = 0
        out[s] = (di, offset)
    return out


class DatasetForCausalLM(torch.utils.data.Dataset):
    def __init__(self, data_name: str, max_seq_length: int, binarization_impl: str = "mmap",
                 split_type: str = "train", start_weight: float = 0.0, end_weight: float = 1.0,
                 seed: Optional[int] = None) -> None:
        if binarization_impl not in ("lazy", "mmap", "cached"):
            raise ValueError("binarization_impl must be one of 'lazy', 'mmap', 'cached'")
        if not (0.0 <= start_weight < 1.0) or not (0.0 < end_weight <= 1.0) or end_weight <= start_weight:
            raise ValueError("need 0 <= start_weight < end_weight <= 1")
        if end_weight - start_weight < 0.1 - 1e-12:
            raise ValueError("end_weight - start_weight must be at least 0.1")
        self.name = data_name
        self.max_seq_length = max_seq_length
        self.index = make_dataset(data_name, binarization_impl)
        n = len(self.index)
        start, end = int(round(start_weight * n)), int(round(end_weight * n))
        self.doc_idx, self.sample_idx, self.shuffle_idx = self._index_mappings(
            data_name, split_type, start, end, np.asarray(self.index.sizes), n, max_seq_length, seed)

    def __len__(self) -> int:
        return self.sample_idx.shape[0] - 1

    def __getitem__(self, idx: int):
        idx = int(self.shuffle_idx[idx])
        d0, o0 = (int(x) for x in self.sample_idx[idx])
        d1, o1 = (int(x) for x in self.sample_idx[idx + 1])
        if d0 == d1:
            sample = self.index.get(int(self.doc_idx[d0]), offset=o0, length=o1 - o0 + 1)
        else:
            parts = [self.index.get(int(self.doc_idx[d0]), offset=o0)]
            parts += [self.index.get(int(self.doc_idx[i])) for i in range(d0 + 1, d1)]
            parts.append(self.index.get(int(self.doc_idx[d1]), length=o1 + 1))
            sample = np.concatenate(parts)
        ids = torch.from_numpy(np.array(sample, dtype=np.int64))
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()}

    # ------------------------------------------------------------------ index construction
    @staticmethod
    def _index_mappings(data_name, split_type, start, end, sizes, num_samples, max_seq_length, seed):
        local_rank = int(os.getenv("LOCAL_RANK", 0))
        world = int(os.getenv("WORLD_SIZE", 1))
        rng = np.random.RandomState(seed if seed is not None else 42)
        docs = np.arange(start, end, dtype=np.int32)
        tokens = int(np.sum(sizes[docs]))
        stem = f"{data_name}_{split_type}_samples={num_samples}_length={max_seq_length}"
        if seed is not None:
            stem += f"_seed={seed}"
        files = [stem + s for s in ("_doc_idx.npy", "_sample_idx.npy", "_shuffle_idx.npy")]
        if local_rank == 0 and not all(os.path.isfile(f) for f in files):
            doc_idx = docs.copy()
            rng.shuffle(doc_idx)
            sizes32 = np.ascontiguousarray(sizes, dtype=np.int32)
            cpp = cpp_builders.load()
            if cpp is not None:
                sample_idx = cpp.build_sample_idx(sizes32, doc_idx, max_seq_length - 1, 1, tokens)
            else:
                sample_idx = build_sample_idx_numpy(sizes32, doc_idx, max_seq_length - 1, 1, tokens)
            total = sample_idx.shape[0] - 1
            dt = np.uint32 if total < np.iinfo(np.uint32).max - 1 else np.int64
            shuffle_idx = np.arange(total, dtype=dt)
            rng.shuffle(shuffle_idx)
            for f, a in zip(files, (doc_idx, sample_idx, shuffle_idx)):
                np.save(f, a, allow_pickle=True)
        if world > 1 and dist.is_available():
            if not dist.is_initialized():
                from ..parallel.mpu import MPU
                MPU.initialize_distributed()
            dist.barrier()
        return tuple(np.load(f, allow_pickle=True, mmap_mode="r") for f in files)
