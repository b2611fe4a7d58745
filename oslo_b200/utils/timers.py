"""Device-side timers (CUDA events on the launching stream) with max-over-ranks reduction, NVTX ranges."""
from __future__ import annotations

import contextlib
import time
from typing import Dict, List

import torch
import torch.distributed as dist


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is present (shows up in profilers), no-op otherwise."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """``with timer("fwd"): ...`` records a CUDA-event pair (wall clock on CPU). ``summary()`` synchronises once."""

    def __init__(self) -> None:
        self._events: Dict[str, List] = {}
        self._wall: Dict[str, List[float]] = {}

    @contextlib.contextmanager
    def __call__(self, name: str):
        if torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            with nvtx_range(name):
                yield
            b.record()
            self._events.setdefault(name, []).append((a, b))
        else:
            t0 = time.perf_counter()
            yield
            self._wall.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)

    def summary(self, group=None, reset: bool = True) -> Dict[str, float]:
        """Mean milliseconds per name; with a process group, the MAX over its ranks."""
        out: Dict[str, float] = {}
        if self._events:
            torch.cuda.synchronize()
        for name, pairs in self._events.items():
            out[name] = sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)
        for name, vals in self._wall.items():
            out[name] = sum(vals) / len(vals)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1 and out:
            names = sorted(out)
            dev = "cuda" if (torch.cuda.is_available() and dist.get_backend(group) == "nccl") else "cpu"
            t = torch.tensor([out[n] for n in names], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out = dict(zip(names, t.tolist()))
        if reset:
            self._events.clear()
            self._wall.clear()
        return out
