"""Weighted interleaving of several datasets (reference: oslo/data/utils/blenders.py:38-117)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from . import cpp_builders


def build_blending_indices_numpy(dataset_index, dataset_sample_index, weights, num_datasets, size) -> None:
    """Greedy max-error assignment (oracle for the C++ builder)."""
    taken = np.zeros(num_datasets, dtype=np.int64)
    w = np.asarray(weights, dtype=np.float64)
    for i in range(size):
        denom = max(float(i), 1.0)
        err = w * denom - taken
        best = int(np.argmax(err))
        dataset_index[i] = best
        dataset_sample_index[i] = taken[best]
        taken[best] += 1


class DatasetBlender(torch.utils.data.Dataset):
    def __init__(self, datasets: Sequence[torch.utils.data.Dataset], weights: Optional[List[float]] = None) -> None:
        if not datasets:
            raise ValueError("no datasets given")
        if len(datasets) >= 255:
            raise ValueError("at most 254 datasets can be blended")
        self.datasets = list(datasets)
        n = len(self.datasets)
        self.size = sum(len(d) for d in self.datasets)
        if weights is None:
            weights = [len(d) / self.size for d in self.datasets]
        if len(weights) != n:
            raise ValueError("weights and datasets differ in length")
        w = np.asarray(weights, dtype=np.float64)
        if w.sum() <= 0:
            raise ValueError("weights must sum to a positive number")
        w = w / w.sum()
        self.weights = w
        self.dataset_index = np.zeros(self.size, dtype=np.uint8)
        self.dataset_sample_index = np.zeros(self.size, dtype=np.int64)
        cpp = cpp_builders.load()
        if cpp is not None:
            cpp.build_blending_indices(self.dataset_index, self.dataset_sample_index, w, n, self.size)
        else:
            build_blending_indices_numpy(self.dataset_index, self.dataset_sample_index, w, n, self.size)

    def __len__(self) -> int:
        return self.size

    def __getitem__(self, idx: int):
        d = int(self.dataset_index[idx])
        s = int(self.dataset_sample_index[idx]) % len(self.datasets[d])
        return self.datasets[d][s]
