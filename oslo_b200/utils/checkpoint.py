"""Training-state sidecar for true resume: optimizer shard, loss scale, step counter and random-number
generators of ONE rank, next to the model files of ``save_pretrained_with_parallel``.

The reference saves weights only (oslo/parallelism_utils.py:431-566); optimizer state is left to whatever
engine wraps the model. One file per rank, ``oslo_state_tp={i}_pp={j}_dp={k}.pt``: the ZeRO-1 shard of
``FusedAdamW`` differs per data-parallel rank, and dropout masks depend on each rank's generator.
"""
from __future__ import annotations

import os
import random
import re
import shutil
from typing import Any, Callable, Dict, List, Optional

import torch

STATE_NAME = "oslo_state_tp={tp}_pp={pp}_dp={dp}.pt"
FORMAT_VERSION = 1


class CheckpointUnreadable(RuntimeError):
    """A checkpoint file exists but cannot be read back (truncated by a crash, damaged on disk)."""


def atomic_save(obj: Any, path: str, save_function: Callable = torch.save) -> None:
    """Write through ``<path>.tmp`` and rename: a crash while writing never leaves a truncated file under the final
    name (the previous file, if any, stays in place until the new one is complete)."""
    tmp = path + ".tmp"
    save_function(obj, tmp)
    try:                                  # the bytes are on the device before the name changes
        fd = os.open(tmp, os.O_RDONLY)
        try:
            os.fsync(fd)
        finally:
            os.close(fd)
    except OSError:
        pass                              # a save_function that wrote elsewhere, or a filesystem without fsync
    os.replace(tmp, path)


def load_file(path: str, weights_only: bool = True) -> Any:
    """``torch.load`` that says which file is unreadable instead of surfacing an unpickling error."""
    try:
        return torch.load(path, map_location="cpu", weights_only=weights_only)
    except FileNotFoundError:
        raise
    except Exception as e:  # noqa: BLE001 - zip / pickle / EOF errors of a damaged file, whatever their class
        raise CheckpointUnreadable(f"{path} cannot be read (truncated or damaged): {type(e).__name__}: {e}") from e


def _coords(mpu) -> Dict[str, int]:
    if mpu is None:
        return dict(tp=0, pp=0, dp=0)
    return dict(tp=mpu.get_tensor_parallel_rank(), pp=mpu.get_pipeline_parallel_rank(),
                dp=mpu.get_data_parallel_rank())


def state_file(directory: str, mpu=None) -> str:
    return os.path.join(directory, STATE_NAME.format(**_coords(mpu)))


def _rng_state() -> Dict[str, Any]:
    st: Dict[str, Any] = dict(torch_cpu=torch.get_rng_state(), python=random.getstate())
    try:
        import numpy as np
        st["numpy"] = np.random.get_state()
    except Exception:  # numpy is optional for the framework proper
        pass
    if torch.cuda.is_available():
        st["torch_cuda"] = torch.cuda.get_rng_state()
    return st


def _set_rng_state(st: Dict[str, Any]) -> None:
    torch.set_rng_state(st["torch_cpu"])
    random.setstate(st["python"])
    if "numpy" in st:
        import numpy as np
        np.random.set_state(st["numpy"])
    if "torch_cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["torch_cuda"])


def save_training_state(directory: str, optimizer=None, step: int = 0, mpu=None,
                        extra: Optional[Dict[str, Any]] = None) -> str:
    """Write this rank's sidecar into ``directory`` (created if missing); returns the path. Call it on every
    rank, after ``model.save_pretrained_with_parallel(directory)``."""
    os.makedirs(directory, exist_ok=True)
    path = state_file(directory, mpu)
    payload = dict(version=FORMAT_VERSION, step=int(step), coords=_coords(mpu), rng=_rng_state(),
                   optimizer=optimizer.state_dict() if optimizer is not None else None, extra=extra or {})
    atomic_save(payload, path)
    return path


def load_training_state(directory: str, optimizer=None, mpu=None, restore_rng: bool = True) -> Dict[str, Any]:
    """Restore optimizer / loss scale / generators of this rank; returns ``{"step": ..., "extra": ...}``.
    The parallel layout must be the one the state was saved with (the optimizer shard is checked)."""
    path = state_file(directory, mpu)
    resharded = _load_resharded(directory, optimizer, mpu)
    if resharded is not None:
        return resharded
    if not os.path.exists(path):
        raise FileNotFoundError(f"no training state for this rank: {path}")
    payload = load_file(path, weights_only=False)
    if payload.get("version") != FORMAT_VERSION:
        raise ValueError(f"{path}: unknown training-state version {payload.get('version')}")
    if payload["coords"] != _coords(mpu):
        raise ValueError(f"{path}: saved for ranks {payload['coords']}, loading on {_coords(mpu)}")
    if optimizer is not None:
        if payload["optimizer"] is None:
            raise ValueError(f"{path} holds no optimizer state")
        optimizer.load_state_dict(payload["optimizer"])
    if restore_rng:
        _set_rng_state(payload["rng"])
    return dict(step=payload["step"], extra=payload["extra"])


def _load_resharded(directory: str, optimizer, mpu) -> Optional[Dict[str, Any]]:
    """The job continues with another number of data-parallel replicas than it was saved with (same tensor / pipeline
    layout): this rank's ZeRO-1 shard is re-cut from the old ranks' sidecars. Returns ``None`` when the saved sharding
    is the current one (or there is nothing to re-cut). Generators are left alone: with another replica count the data
    order changes anyway, so such a resume is exact in the optimizer state but not bit for bit in what follows."""
    if optimizer is None or not hasattr(optimizer, "reshard_state"):
        return None
    c = _coords(mpu)
    first = os.path.join(directory, STATE_NAME.format(tp=c["tp"], pp=c["pp"], dp=0))
    if not os.path.exists(first):
        return None
    head = load_file(first, weights_only=False)
    old_opt = head.get("optimizer")
    if old_opt is None or int(old_opt["shards"]) == int(optimizer.shards):
        return None
    n_old, old_shards = old_opt["master"].numel(), int(old_opt["shards"])
    lo, hi = optimizer.shard_rank * optimizer.shard_numel, (optimizer.shard_rank + 1) * optimizer.shard_numel
    states = []
    for r in range(old_shards):
        if r * n_old < hi and (r + 1) * n_old > lo:
            f = os.path.join(directory, STATE_NAME.format(tp=c["tp"], pp=c["pp"], dp=r))
            states.append(old_opt if r == 0 else load_file(f, weights_only=False)["optimizer"])
    sd = optimizer.reshard_state(states or [old_opt], optimizer.shards, optimizer.shard_rank, optimizer.shard_numel)
    optimizer.load_state_dict(sd)
    return dict(step=head["step"], extra=head["extra"], resharded_from=old_shards)


# ---------------------------------------------------------------------------------------------------------------
# Checkpoint generations with a "latest" pointer: what a job that may die at any moment resumes from.

def rank_coords(rank: int, world: int, tp: int, pp: int) -> Dict[str, int]:
    """(tp, pp, dp) coordinates of a global rank in the ``MPU`` layout, computable before any model exists."""
    per_stage = world // pp
    return dict(tp=rank % tp, pp=rank // per_stage, dp=(rank % per_stage) // tp)


class CheckpointManager:
    """``<root>/step-00000200/`` directories (model files of ``save_pretrained_with_parallel`` + every rank's
    training-state sidecar) and ``<root>/latest``, a one-line file naming the newest COMPLETE generation.

    ``save`` is collective: all ranks write their files, meet, and only then rank 0 moves the pointer (atomically) and
    removes generations beyond ``keep``. A job that dies in the middle of a save therefore leaves the pointer on the
    previous generation. ``latest_usable`` is collective too: every rank reads back its own files of the newest
    generation, the ranks agree (all-reduce) whether all of them succeeded, and fall back generation by generation
    otherwise - a damaged shard on one rank sends all ranks to the older checkpoint together. The reference has no
    counterpart (it writes weights into one directory, oslo/parallelism_utils.py:431-566)."""

    POINTER = "latest"
    _STEP = re.compile(r"^step-(\d{8})$")

    def __init__(self, root: str, keep: int = 2) -> None:
        self.root, self.keep = root, max(1, int(keep))

    # -- helpers
    @staticmethod
    def _rank_world():
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
        return 0, 1

    @staticmethod
    def _barrier() -> None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.barrier()

    def step_dir(self, step: int) -> str:
        return os.path.join(self.root, f"step-{int(step):08d}")

    def generations(self) -> List[str]:
        """Existing generation directories, newest first."""
        if not os.path.isdir(self.root):
            return []
        names = sorted((n for n in os.listdir(self.root) if self._STEP.match(n)), reverse=True)
        return [os.path.join(self.root, n) for n in names]

    def pointer(self) -> Optional[str]:
        """Directory the ``latest`` file names, or ``None`` (no pointer, or it names something that is gone)."""
        try:
            with open(os.path.join(self.root, self.POINTER)) as f:
                name = f.read().strip()
        except OSError:
            return None
        d = os.path.join(self.root, name)
        return d if (self._STEP.match(name) and os.path.isdir(d)) else None

    # -- saving
    def save(self, model, optimizer=None, step: int = 0, extra: Optional[Dict[str, Any]] = None) -> str:
        d = self.step_dir(step)
        model.save_pretrained_with_parallel(d)
        model.save_training_state(d, optimizer, step=step, extra=extra)
        self._barrier()                                # every rank's files of this generation are complete
        rank, _ = self._rank_world()
        if rank == 0:
            tmp = os.path.join(self.root, self.POINTER + ".tmp")
            with open(tmp, "w") as f:
                f.write(os.path.basename(d) + "\n")
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, os.path.join(self.root, self.POINTER))
            for old in self.generations()[self.keep:]:
                shutil.rmtree(old, ignore_errors=True)
        self._barrier()
        return d

    # -- resuming
    def _readable_here(self, directory: str, tp: int, pp: int) -> bool:
        """This rank's model file and sidecar of ``directory`` load back."""
        from ..parallelism_utils import WEIGHTS_NAME_PARALLEL
        rank, world = self._rank_world()
        c = rank_coords(rank, world, tp, pp)
        model_file = (os.path.join(directory, WEIGHTS_NAME_PARALLEL.format(tp=c["tp"], pp=c["pp"]))
                      if tp * pp > 1 else os.path.join(directory, "pytorch_model.bin"))
        own = os.path.join(directory, STATE_NAME.format(**c))
        if not os.path.exists(own):      # saved with fewer data-parallel replicas: the shards get re-cut from theirs
            own = os.path.join(directory, STATE_NAME.format(tp=c["tp"], pp=c["pp"], dp=0))
        try:
            load_file(model_file, weights_only=True)
            load_file(own, weights_only=False)
            return os.path.isfile(os.path.join(directory, "config.json"))
        except (OSError, CheckpointUnreadable):
            return False

    def latest_usable(self, tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1) -> Optional[str]:
        """Newest generation that EVERY rank can read (the pointer's first, then older ones), or ``None``."""
        import torch.distributed as dist
        tp, pp = int(tensor_parallel_size), int(pipeline_parallel_size)
        first = self.pointer()
        order = ([first] if first else []) + [g for g in self.generations() if g != first and (first is None or g < first)]
        for d in order:
            ok = torch.tensor([1 if self._readable_here(d, tp, pp) else 0])
            if dist.is_available() and dist.is_initialized():
                if dist.get_backend() == "nccl":
                    ok = ok.cuda()
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 1:
                return d
        return None
