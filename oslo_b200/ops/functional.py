"""Public op functions: dispatch between the sm_100a kernels and the PyTorch statements."""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from . import reference as ref

_GELU_NAMES = ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh")


def _k(x: Tensor) -> bool:
    from . import use_kernels
    return use_kernels(x)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, reversed: bool = False,
           activation: Optional[str] = None) -> Tensor:
    """``act(x @ W.T + b)`` (or ``x @ W`` when ``reversed``). bf16/fp16 CUDA inputs use the tcgen05 GEMM."""
    if _k(x):
        from . import cuda_ops
        return cuda_ops.linear(x, weight, bias, reversed, activation)
    return ref.linear(x, weight, bias, reversed, activation)


def layer_norm(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float = 1e-5) -> Tensor:
    if _k(x):
        from . import cuda_ops
        return cuda_ops.layer_norm(x, weight, bias, eps)
    return ref.layer_norm(x, weight, bias, eps)


def bias_gelu(x: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    if _k(x):
        from . import cuda_ops
        return cuda_ops.bias_gelu(x, bias)
    return ref.bias_gelu(x, bias)


def bias_dropout_residual(x: Tensor, bias: Optional[Tensor] = None, residual: Optional[Tensor] = None,
                          p: float = 0.0, training: bool = False) -> Tensor:
    if _k(x):
        from . import cuda_ops
        return cuda_ops.bias_dropout_residual(x, bias, residual, p, training)
    return ref.bias_dropout_residual(x, bias, residual, p, training)


def rotary_interleaved(x: Tensor, positions: Tensor, rotary_dim: int, base: float = 10000.0) -> Tensor:
    """GPT-J rotary on ``[B, S, heads, D]`` with integer ``positions`` ``[B, S]``."""
    if _k(x):
        from . import cuda_ops
        return cuda_ops.rotary_interleaved(x, positions, rotary_dim, base)
    return ref.rotary_interleaved(x, positions, rotary_dim, base)


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, window: Optional[int] = None,
              scale: Optional[float] = None, key_padding_mask: Optional[Tensor] = None,
              dropout_p: float = 0.0, training: bool = False) -> Tensor:
    """Flash-style attention on ``[B, heads, S, D]`` (any strides with contiguous ``D``)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.size(-1))
    if _k(q) and not (dropout_p > 0.0 and training):
        from . import cuda_ops
        if cuda_ops.flash_supported(q, k, v):
            return cuda_ops.flash_attention(q, k, v, causal, window, scale, key_padding_mask)
    return ref.attention(q, k, v, causal, window, scale, key_padding_mask, dropout_p, training)


def decode_attention(q: Tensor, k_cache: Tensor, v_cache: Tensor, lengths: Tensor, scale: float,
                     window: Optional[int] = None) -> Tensor:
    """One-query attention over a static KV cache.

    ``q``: ``[B, heads, D]``; caches ``[B, heads, T_max, D]``; ``lengths``: ``[B]`` valid keys per row
    (the query sits at position ``lengths - 1``).
    """
    if _k(q):
        from . import cuda_ops
        return cuda_ops.decode_attention(q, k_cache, v_cache, lengths, scale, window)
    B, H, T, D = k_cache.shape
    s = torch.einsum("bhd,bhtd->bht", q.float(), k_cache.float()) * scale
    pos = torch.arange(T, device=q.device)[None, :]
    keep = pos < lengths[:, None]
    if window is not None:
        keep &= pos > (lengths[:, None] - 1 - window)
    s = s.masked_fill(~keep[:, None, :], torch.finfo(torch.float32).min)
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bht,bhtd->bhd", p, v_cache.float()).to(q.dtype)


def scaled_upper_triang_masked_softmax(x: Tensor, scale: float = 1.0) -> Tensor:
    if _k(x):
        from . import cuda_ops
        return cuda_ops.causal_softmax(x, scale)
    return _RefCausalSoftmax.apply(x, scale)


def scaled_masked_softmax(x: Tensor, mask: Tensor, scale: float = 1.0) -> Tensor:
    if _k(x):
        from . import cuda_ops
        return cuda_ops.masked_softmax(x, mask, scale)
    return ref.scaled_masked_softmax(x, mask, scale)


class _RefCausalSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        y = ref.scaled_upper_triang_masked_softmax(x, scale)
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return ref.softmax_backward(y, dy, ctx.scale), None


def cross_entropy(logits: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
    """Mean cross-entropy over rows of ``[N, V]`` logits with fp32 math."""
    if _k(logits):
        from . import cuda_ops
        return cuda_ops.cross_entropy(logits, labels, ignore_index)
    return ref.cross_entropy(logits, labels, ignore_index)


def linear_cross_entropy(hidden: Tensor, weight: Tensor, bias: Optional[Tensor], labels: Tensor,
                         ignore_index: int = -100, chunk_rows: int = 4096) -> Tensor:
    """LM-head projection fused with the loss, never holding more than ``chunk_rows`` rows of logits.

    ``hidden``: ``[N, H]``, ``weight``: ``[V, H]``, ``labels``: ``[N]`` (already shifted). Returns the
    mean loss over rows whose label is not ``ignore_index``.
    """
    if _k(hidden):
        from . import cuda_ops
        return cuda_ops.linear_cross_entropy(hidden, weight, bias, labels, ignore_index, chunk_rows)
    logits = ref.linear(hidden, weight, bias)
    return ref.cross_entropy(logits, labels, ignore_index)


def ban_repeated_ngrams(tokens: Tensor, lprobs: Tensor, n: int) -> Tensor:
    if _k(lprobs):
        from . import cuda_ops
        return cuda_ops.ban_repeated_ngrams(tokens, lprobs, n)
    return ref.ban_repeated_ngrams(tokens, lprobs, n)
