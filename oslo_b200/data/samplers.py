"""Distributed wrapper around any sampler (reference: oslo/data/utils/samplers.py:9-75)."""
from __future__ import annotations

from operator import itemgetter
from typing import Iterator, Optional

from torch.utils.data import Dataset, DistributedSampler, Sampler


class DatasetFromSampler(Dataset):
    """Materialises a sampler's indices so they can themselves be sharded."""

    def __init__(self, sampler: Sampler) -> None:
        self.sampler = sampler
        self.sampler_list = None

    def __getitem__(self, index: int):
        if self.sampler_list is None:
            self.sampler_list = list(self.sampler)
        return self.sampler_list[index]

    def __len__(self) -> int:
        return len(self.sampler)


class DistributedProxySampler(DistributedSampler):
    """Shards the index stream of ``sampler`` over ``num_replicas`` ranks (each rank sees a disjoint part)."""

    def __init__(self, sampler: Sampler, num_replicas: Optional[int] = None, rank: Optional[int] = None,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = False) -> None:
        super().__init__(DatasetFromSampler(sampler), num_replicas=num_replicas, rank=rank, shuffle=shuffle,
                         seed=seed, drop_last=drop_last)
        self.sampler = sampler

    def __iter__(self) -> Iterator[int]:
        self.dataset = DatasetFromSampler(self.sampler)
        positions = list(super().__iter__())
        if not positions:
            return iter([])
        got = itemgetter(*positions)(self.dataset)
        return iter(got if isinstance(got, tuple) else (got,))
