"""Loader that restarts its iterator instead of stopping (reference: oslo/data/utils/loaders.py:4-24)."""
from __future__ import annotations


class InfiniteDataLoader:
    def __init__(self, loader) -> None:
        self.loader = loader
        self.iterator = iter(loader)
        self.epoch = 0

    def __iter__(self):
        return self

    def __next__(self):
        try:
            return next(self.iterator)
        except StopIteration:
            self.epoch += 1
            sampler = getattr(self.loader, "sampler", None)
            if hasattr(sampler, "set_epoch"):
                sampler.set_epoch(self.epoch)
            self.iterator = iter(self.loader)
            return next(self.iterator)
