"""Op layer: every function has a PyTorch statement (``reference``) and an sm_100a kernel path.

Dispatch rule: CUDA tensors go to the hand-written kernels of the in-tree extension
(``oslo_b200/_C.so``); CPU tensors go to the PyTorch statement. A CUDA tensor with no
loadable extension is an error unless ``OSLO_B200_ALLOW_FALLBACK=1`` is set, so a GPU run
can never silently execute the library path.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
from torch import Tensor

from . import reference

_EXT = None
_EXT_ERR: Optional[BaseException] = None


def ext_path() -> str:
    """``_C.so``, or with ``OSLO_B200_DEBUG_BOUNDS=1`` the debug build ``_C_bounds.so`` (``python -m oslo_b200.build
    --debug-bounds``): the same kernels compiled with ``-DOSLO_DEBUG_BOUNDS``, which record ``ERR_BOUNDS`` in the device
    error word whenever a data-dependent index (token id, cache position, sequence length) had to be skipped or clamped."""
    name = "_C_bounds.so" if os.environ.get("OSLO_B200_DEBUG_BOUNDS", "0").lower() in ("1", "true", "yes", "on") else "_C.so"
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), name)


def load_ext(required: bool = False):
    """Load the prebuilt extension once. Returns the ``torch.ops.oslo_b200`` namespace or None."""
    global _EXT, _EXT_ERR
    if _EXT is None and _EXT_ERR is None:
        try:
            path = ext_path()
            if not os.path.exists(path):
                raise FileNotFoundError(f"{path} not built; run `python -m oslo_b200.build`")
            torch.ops.load_library(path)
            _EXT = torch.ops.oslo_b200
            try:   # shape / dtype implementations for graph capture; never fatal
                from . import fake_impls
                fake_impls.register()
            except Exception:  # noqa: BLE001
                pass
        except BaseException as e:  # noqa: BLE001 - reported below
            _EXT_ERR = e
    if _EXT is None and required:
        raise RuntimeError(f"oslo_b200 CUDA extension unavailable: {_EXT_ERR!r}")
    return _EXT


def kernels_available() -> bool:
    return torch.cuda.is_available() and load_ext() is not None


def use_kernels(x: Tensor) -> bool:
    """True when ``x`` must run on the sm_100a kernels."""
    if not x.is_cuda:
        return False
    if load_ext() is not None:
        return True
    if os.environ.get("OSLO_B200_ALLOW_FALLBACK") == "1":
        return False
    raise RuntimeError(
        "CUDA tensor given but the oslo_b200 extension is not loadable "
        f"({_EXT_ERR!r}); build it with `python -m oslo_b200.build` or set OSLO_B200_ALLOW_FALLBACK=1"
    )


from .functional import (  # noqa: E402
    linear, layer_norm, bias_gelu, bias_dropout_residual, rotary_interleaved, attention,
    scaled_upper_triang_masked_softmax, scaled_masked_softmax, cross_entropy, linear_cross_entropy,
    ban_repeated_ngrams, decode_attention,
)

__all__ = [
    "reference", "load_ext", "kernels_available", "use_kernels", "linear", "layer_norm", "bias_gelu",
    "bias_dropout_residual", "rotary_interleaved", "attention", "scaled_upper_triang_masked_softmax",
    "scaled_masked_softmax", "cross_entropy", "linear_cross_entropy", "ban_repeated_ngrams",
    "decode_attention",
]
