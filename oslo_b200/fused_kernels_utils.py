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
    cross-attention; the training path uses flash attention and never materialises scores).
    Argument order as in the reference (oslo/fused_kernels_utils.py:431-479)."""

    @staticmethod
    def is_available(dtype, bsz: int, np: int, sq: int, sk: int, use_triang_mask: bool) -> bool:
        """The reference's kernels take fp16 scores of at most 2048 keys in batch-per-block multiples; the softmax
        kernels here are one block per row with no such limits, so only the shape has to make sense."""
        if dtype not in (torch.float16, torch.bfloat16, torch.float32) or min(bsz, np, sq, sk) <= 0:
            return False
        return (sq == sk) if use_triang_mask else True

    @staticmethod
    def apply(input: Tensor, pad_mask: Optional[Tensor], scale: Optional[float], use_triang_mask: bool) -> Tensor:
        """``input``: ``[b, heads, sq, sk]`` scores. With ``use_triang_mask`` the causal mask is applied by the kernel
        and ``pad_mask`` (optional) is either an additive float mask, as the reference passes it, or a boolean /
        uint8 mask with 1 = masked. Without it ``pad_mask`` is boolean / uint8 with 1 = masked, broadcastable to
        ``[b, 1, sq, sk]``; ``None`` masks nothing."""
        from . import ops
        b, h, sq, sk = input.shape
        scale = 1.0 if scale is None else float(scale)
        if use_triang_mask:
            if pad_mask is not None:
                if pad_mask.is_floating_point():
                    input = input + pad_mask
                else:
                    input = input.masked_fill(pad_mask.to(torch.bool), -10000.0 / max(scale, 1e-20))
            return ops.scaled_upper_triang_masked_softmax(input.reshape(b * h, sq, sk), scale).view(b, h, sq, sk)
        if pad_mask is None:
            pad_mask = torch.zeros(b, 1, sq, sk, dtype=torch.uint8, device=input.device)
        elif pad_mask.shape[-2] != sq or pad_mask.shape[0] != b:
            pad_mask = pad_mask.expand(b, 1, sq, sk)
        return ops.scaled_masked_softmax(input, pad_mask.to(torch.uint8).contiguous(), scale)


class FusedBiasActivation:
    @staticmethod
    def apply(x: Tensor, bias: Optional[Tensor], act: str = "gelu_new") -> Tensor:
        from . import ops
        if act in ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh"):
            return ops.bias_gelu(x, bias)
        y = x if bias is None else x + bias
        return ACT2FN[act](y)


class FusedBiasDropout:
    """``apply(x, bias, training, drop_prop)`` (reference: oslo/fused_kernels_utils.py:399-412)."""

    @staticmethod
    def apply(x: Tensor, bias: Optional[Tensor], training: bool, drop_prop: float) -> Tensor:
        return bias_dropout(x, bias, drop_prop, training)


class FusedBiasDropoutResidual:
    """``apply(x, bias, residual, training, drop_prop)`` (reference: oslo/fused_kernels_utils.py:415-428)."""

    @staticmethod
    def apply(x: Tensor, bias: Optional[Tensor], residual: Tensor, training: bool, drop_prop: float) -> Tensor:
        return bias_dropout_residual(x, bias, residual, drop_prop, training)


# ---------------------------------------------------------------------- function-style entry points of the reference
# (oslo/fused_kernels_utils.py:260-380): there they are TorchScript-fused elementwise chains and autograd wrappers
# around three CUDA kernels; here each is one call of the corresponding kernel (or its PyTorch statement on CPU).
def bias_dropout(x: Tensor, bias: Optional[Tensor], prob: float, training: bool) -> Tensor:
    from . import ops
    return ops.bias_dropout_residual(x, bias, None, float(prob), bool(training))


def bias_dropout_train(x: Tensor, bias: Optional[Tensor], prob: float) -> Tensor:
    return bias_dropout(x, bias, prob, True)


def bias_dropout_inference(x: Tensor, bias: Optional[Tensor], prob: float) -> Tensor:
    return bias_dropout(x, bias, prob, False)


def bias_dropout_residual(x: Tensor, bias: Optional[Tensor], residual: Tensor, prob: float, training: bool) -> Tensor:
    from . import ops
    return ops.bias_dropout_residual(x, bias, residual, float(prob), bool(training))


def bias_dropout_residual_train(x: Tensor, bias: Optional[Tensor], residual: Tensor, prob: float) -> Tensor:
    return bias_dropout_residual(x, bias, residual, prob, True)


def bias_dropout_residual_inference(x: Tensor, bias: Optional[Tensor], residual: Tensor, prob: float) -> Tensor:
    return bias_dropout_residual(x, bias, residual, prob, False)


def bias_gelu_fwb(y: Tensor, bias: Optional[Tensor]) -> Tensor:
    """tanh-GeLU of ``y + bias`` (the forward half; the name is the reference's)."""
    from .ops import reference
    return reference.bias_gelu(y, bias)


def bias_gelu_bwd(g: Tensor, y: Tensor, bias: Optional[Tensor]) -> Tensor:
    """Gradient of ``bias_gelu_fwb`` with respect to ``y`` (and, summed over rows, to ``bias``)."""
    x = (y if bias is None else y + bias).float()
    t = torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x))
    dx = 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * 0.7978845608028654 * (1.0 + 3.0 * 0.044715 * x * x)
    return (g.float() * dx).to(g.dtype)


class FusedBiasGeLU:
    """``FusedBiasGeLU.apply(input, bias)``: bias + tanh-GeLU with its backward, one kernel each way on GPUs."""

    @staticmethod
    def apply(input: Tensor, bias: Optional[Tensor]) -> Tensor:
        from . import ops
        return ops.bias_gelu(input, bias)


class ScaledUpperTriangMaskedSoftmaxFunction:
    """``apply(inputs [batch * heads, sq, sk], scale)``: causal softmax with autograd."""

    @staticmethod
    def apply(inputs: Tensor, scale: float) -> Tensor:
        from . import ops
        return ops.scaled_upper_triang_masked_softmax(inputs, float(scale))


class ScaledMaskedSoftmaxFunction:
    """``apply(inputs [b, heads, sq, sk], mask (1 = masked), scale)``: masked softmax with autograd."""

    @staticmethod
    def apply(inputs: Tensor, mask: Tensor, scale: float) -> Tensor:
        from . import ops
        b, _h, sq, sk = inputs.shape
        return ops.scaled_masked_softmax(inputs, mask.expand(b, 1, sq, sk).to(torch.uint8).contiguous(), float(scale))


class NGramRepeatBlockFunction:
    """``apply(tokens, lprobs, bsz, step, beam_size, no_repeat_ngram_size)``: ``-inf`` on every token that would repeat
    an n-gram of its row, in place (no gradient). ``tokens`` holds ``step + 1`` generated tokens per row; ``bsz``,
    ``step`` and ``beam_size`` are implied by the shapes and only accepted for call compatibility."""

    @staticmethod
    def apply(tokens: Tensor, lprobs: Tensor, bsz: int, step: int, beam_size: int, no_repeat_ngram_size: int) -> Tensor:
        from . import ops
        return ops.ban_repeated_ngrams(tokens, lprobs, int(no_repeat_ngram_size))


class AbstractKernelBuilder:
    """Build-and-load handle with the reference's interface (oslo/fused_kernels_utils.py:53-181). The reference JIT
    compiles at first use for whatever architecture it finds; here everything is compiled ahead of time for sm_100a
    by ``oslo_b200.build`` and ``load()`` only (re)builds when sources changed."""

    @property
    def base_path(self) -> str:
        import os
        return os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")

    @property
    def name(self) -> str:
        raise NotImplementedError

    def sources(self):
        raise NotImplementedError

    def includes(self):
        return [self.base_path]

    @staticmethod
    def get_compatibility_version() -> str:
        return "10.0a"

    @staticmethod
    def cxx_args():
        return ["-O3", "-std=c++17", "-fPIC"]

    def nvcc_args(self, maxrregcount: Optional[int] = None):
        from . import build
        return list(build.NVCC_FLAGS) + ([f"-maxrregcount={int(maxrregcount)}"] if maxrregcount else [])

    def load(self):
        raise NotImplementedError


class KernelBuilder(AbstractKernelBuilder):
    name = "oslo_b200._C"

    def sources(self):
        import os
        from . import build
        return [os.path.join(self.base_path, f) for f in build.CUDA_SOURCES + build.CPP_SOURCES]

    def load(self):
        from . import build, ops
        build.build_kernels(force=False, verbose=False)
        return ops.load_ext(required=True)


class DatasetsBuilder(AbstractKernelBuilder):
    name = "oslo_b200._data_C"

    def sources(self):
        import os
        return [os.path.join(self.base_path, "data_builders.cpp")]

    def load(self):
        from . import build
        from .data import cpp_builders
        build.build_data(force=False, verbose=False)
        return cpp_builders.load()


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
