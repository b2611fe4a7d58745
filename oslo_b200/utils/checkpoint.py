"""Training-state sidecar for true resume: optimizer shard, loss scale, step counter and random-number
generators of ONE rank, next to the model files of ``save_pretrained_with_parallel``.

The reference saves weights only (oslo/parallelism_utils.py:431-566); optimizer state is left to whatever
engine wraps the model. One file per rank, ``oslo_state_tp={i}_pp={j}_dp={k}.pt``: the ZeRO-1 shard of
``FusedAdamW`` differs per data-parallel rank, and dropout masks depend on each rank's generator.
"""
from __future__ import annotations

import os
import random
from typing import Any, Dict, Optional

import torch

STATE_NAME = "oslo_state_tp={tp}_pp={pp}_dp={dp}.pt"
FORMAT_VERSION = 1


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
    tmp = path + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, path)   # a crash while writing never leaves a truncated sidecar under the final name
    return path


def load_training_state(directory: str, optimizer=None, mpu=None, restore_rng: bool = True) -> Dict[str, Any]:
    """Restore optimizer / loss scale / generators of this rank; returns ``{"step": ..., "extra": ...}``.
    The parallel layout must be the one the state was saved with (the optimizer shard is checked)."""
    path = state_file(directory, mpu)
    if not os.path.exists(path):
        raise FileNotFoundError(f"no training state for this rank: {path}")
    payload = torch.load(path, map_location="cpu", weights_only=False)
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
