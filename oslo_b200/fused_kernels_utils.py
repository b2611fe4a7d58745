"""``model.fuse()`` and the fused-op helper classes.

``fuse()`` switches a model from library PyTorch ops to this package's sm_100a kernels: modules
named by each layer policy's ``fused_modules()`` get their class swapped to the fused subclass
(exact-class matches only, so e.g. GPT-Neo's local-attention subclass can be mapped separately),
and every linear / norm building block is flagged to dispatch to ``oslo_b200.ops``
(reference: oslo/fused_kernels_utils.py:524-566). The extension is built ahead of time
(``python -m oslo_b200.build``), never at first call.
"""
from __future__ import annotations

import logging
from typing import Iterable, Optional

import torch
from torch import Tensor

logger = logging.getLogger(__name__)


def get_custom_kernels():
    """The loaded kernel namespace (``torch.ops.oslo_b200``); raises if it cannot be loaded."""
    from . import ops
    return ops.load_ext(required=True)


def get_datasets_builder():
    """C++ dataset index builders, or ``None`` when the host extension is not built."""
    from .data import cpp_builders
    return cpp_builders.load()


class FusedKernelMixin:
    def fuse(self, modules: Optional[Iterable[type]] = None):
        """Switch to the fused kernels; ``modules`` restricts the class swap to a subset of the
        policy's fusable classes (e.g. ``model.fuse([GPT2MLP])``). Returns the model."""
        if not getattr(self, "is_fusable", True):
            raise RuntimeError(f"{type(self).__name__} is not fusable")
        mapping = {}
        for policy in self.get_layer_policies():
            mapping.update(policy.fused_modules())
        if modules is not None:
            modules = list(modules)
            unknown = [m for m in modules if m not in mapping]
            if unknown:
                raise ValueError(
                    f"cannot fuse {[m.__name__ for m in unknown]}; fusable: {[m.__name__ for m in mapping]}")
            mapping = {k: v for k, v in mapping.items() if k in modules}
        for m in self.modules():
            cls = type(m)
            if cls in mapping:
                m.__class__ = mapping[cls]
                m.config = self.config
            if hasattr(cls, "oslo_fused") and modules is None:
                m.oslo_fused = True
        self._oslo_fused = True
        return self

    def is_fused(self) -> bool:
        return bool(getattr(self, "_oslo_fused", False))


class FusedScaleMaskSoftmax:
    """Scale + mask + softmax on materialised scores (kept for ``output_attentions=True`` and
    cross-attention; the training path uses flash attention and never materialises scores)."""

    @staticmethod
    def is_available(scores: Tensor, use_triang_mask: bool) -> bool:
        return scores.dim() == 4 and scores.size(-1) > 0 and (not use_triang_mask or scores.size(-1) == scores.size(-2))

    @staticmethod
    def apply(scores: Tensor, scale: float = 1.0, use_triang_mask: bool = True, pad_mask: Optional[Tensor] = None):
        """``scores``: ``[b, heads, sq, sk]``. ``pad_mask`` uint8/bool with 1 = masked."""
        from . import ops
        b, h, sq, sk = scores.shape
        if use_triang_mask:
            if pad_mask is not None:
                scores = scores.masked_fill(pad_mask.to(torch.bool), -10000.0 / max(scale, 1e-20))
            return ops.scaled_upper_triang_masked_softmax(scores.reshape(b * h, sq, sk), scale).view(b, h, sq, sk)
        if pad_mask is None:
            pad_mask = torch.zeros(b, 1, sq, sk, dtype=torch.uint8, device=scores.device)
        return ops.scaled_masked_softmax(scores, pad_mask, scale)


class FusedBiasActivation:
    @staticmethod
    def apply(x: Tensor, bias: Optional[Tensor], act: str = "gelu_new") -> Tensor:
        from . import ops
        if act in ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh"):
            return ops.bias_gelu(x, bias)
        y = x if bias is None else x + bias
        return ACT2FN[act](y)


class FusedBiasDropout:
    @staticmethod
    def apply(x: Tensor, bias: Optional[Tensor], p: float, training: bool) -> Tensor:
        from . import ops
        return ops.bias_dropout_residual(x, bias, None, p, training)


class FusedBiasDropoutResidual:
    @staticmethod
    def apply(x: Tensor, bias: Optional[Tensor], residual: Tensor, p: float, training: bool) -> Tensor:
        from . import ops
        return ops.bias_dropout_residual(x, bias, residual, p, training)


def _gelu_new(x: Tensor) -> Tensor:
    from .ops import reference
    return reference.gelu_tanh(x)


ACT2FN = {
    "gelu": torch.nn.functional.gelu,
    "gelu_new": _gelu_new,
    "gelu_tanh": _gelu_new,
    "gelu_pytorch_tanh": _gelu_new,
    "relu": torch.nn.functional.relu,
    "silu": torch.nn.functional.silu,
    "swish": torch.nn.functional.silu,
    "tanh": torch.tanh,
}

GELU_TANH_NAMES = ("gelu_new", "gelu_tanh", "gelu_pytorch_tanh")
