"""Building-block modules: plain and tensor-parallel linear / embedding / norm layers.

Every module carries ``oslo_fused``: ``False`` runs library PyTorch ops (the state before
``model.fuse()``), ``True`` runs the sm_100a kernels of ``oslo_b200.ops``. The tensor-parallel
classes are installed by swapping ``module.__class__`` after the weights were sliced, so
``state_dict`` keys never change (reference: oslo/modeling_utils.py:15-104,
oslo/parallelism/engine_tensor.py:439-446).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import ops
from .mpu import ceil_split_sizes


_GELU_NAMES = ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh")


def _linear(x: Tensor, weight: Tensor, bias: Optional[Tensor], reversed: bool, fused: bool,
            activation: Optional[str] = None, residual: Optional[Tensor] = None) -> Tensor:
    if fused and residual is not None and x.is_cuda:
        from ..ops import cuda_ops
        return cuda_ops.linear(x, weight, bias, reversed, activation, residual)
    y = ops.linear(x, weight, bias, reversed, activation) if fused else ops.reference.linear(x, weight, bias, reversed, activation)
    return y if residual is None else y + residual


class Linear(nn.Linear):
    """``nn.Linear`` (weight ``[out, in]``) with an optional fused activation epilogue."""

    oslo_fused = False
    reversed = False

    def forward(self, x: Tensor, activation: Optional[str] = None, residual: Optional[Tensor] = None) -> Tensor:
        """``residual`` is added to the result (inside the GEMM epilogue on the kernel path)."""
        return _linear(x, self.weight, self.bias, False, self.oslo_fused, activation, residual)


class Conv1D(nn.Module):
    """GPT-2 style projection with weight stored ``[in, out]``."""

    oslo_fused = False
    reversed = True

    def __init__(self, nf: int, nx: int) -> None:
        super().__init__()
        self.nf = nf
        self.weight = nn.Parameter(torch.empty(nx, nf))
        self.bias = nn.Parameter(torch.zeros(nf))
        nn.init.normal_(self.weight, std=0.02)

    @property
    def in_features(self) -> int:
        return self.weight.size(0)

    @property
    def out_features(self) -> int:
        return self.weight.size(1)

    def forward(self, x: Tensor, activation: Optional[str] = None) -> Tensor:
        return _linear(x, self.weight, self.bias, True, self.oslo_fused, activation)


class LayerNorm(nn.LayerNorm):
    oslo_fused = False

    def forward(self, x: Tensor) -> Tensor:
        if self.oslo_fused:
            return ops.layer_norm(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)


class Embedding(nn.Embedding):
    oslo_fused = False


class VocabParallelEmbedding(nn.Embedding):
    """Embedding whose rows are split over the tensor-parallel group (``torch.chunk`` row ranges).

    Ids outside this rank's range contribute zero rows; the all-reduce over the group restores
    the full lookup (reference: oslo/modeling_utils.py:15-64).
    """

    oslo_fused = False
    mpu = None
    full_num_embeddings: Optional[int] = None

    def vocab_range(self):
        total = self.full_num_embeddings or self.num_embeddings * self.mpu.tp
        sizes = ceil_split_sizes(total, self.mpu.tp)
        start = sum(sizes[: self.mpu.tp_rank])
        return start, start + sizes[self.mpu.tp_rank]

    def forward(self, ids: Tensor) -> Tensor:
        if self.mpu is None or self.mpu.tp == 1:
            return F.embedding(ids, self.weight, self.padding_idx)
        lo, hi = self.vocab_range()
        if self.oslo_fused and ids.is_cuda and self.mpu.backend == "nccl" and self.padding_idx is None:
            from ..config import get_config
            from .symmetric import get_workspace, group_on_one_node, vocab_embed, vocab_embed_usable
            if (get_config().fused_tp_comm and get_config().fused_vocab_embed and ops.kernels_available()
                    and group_on_one_node(self.mpu.get_tensor_parallel_group())):
                ws = get_workspace(self.mpu.get_tensor_parallel_group())
                if vocab_embed_usable(ws, ids, self.weight):
                    return vocab_embed(ws, ids, self.weight, lo, hi)   # lookup + collective in one kernel
        outside = (ids < lo) | (ids >= hi)
        local = (ids - lo).masked_fill(outside, 0)
        out = F.embedding(local, self.weight)
        out = out.masked_fill(outside.unsqueeze(-1), 0.0)
        return self.mpu.reduce(out)


class ColumnParallelLinear(nn.Linear):
    """Linear layer whose output features are split over the tensor-parallel group.

    forward: ``broadcast`` (identity / all-reduce in backward) -> GEMM -> optional gather -> bias.
    With ``parallel=False`` and a ``tied_embedding`` it is the tied LM head of a vocab-parallel
    embedding: the local product yields a vocabulary shard (reference: oslo/modeling_utils.py:67-84).
    """

    oslo_fused = False
    mpu = None
    reversed = False
    gather_output = False
    sequence_parallel = False
    full_out_features: Optional[int] = None

    def forward(self, x: Tensor, activation: Optional[str] = None) -> Tensor:
        mpu = self.mpu
        if self.oslo_fused and not self.gather_output and activation in (None,) + _GELU_NAMES:
            from . import fused_tp
            n_out = self.weight.size(1) if self.reversed else self.weight.size(0)
            rows = x.numel() // max(x.size(-1), 1) * (mpu.tp if (mpu is not None and self.sequence_parallel) else 1)
            if fused_tp.fused_tp_usable(mpu, x, n_out, rows) and (not self.sequence_parallel or rows % (mpu.tp * 128) == 0):
                tp = fused_tp.get_fused_tp(mpu.get_tensor_parallel_group())
                fn = fused_tp._ColumnParallelSeqFused if self.sequence_parallel else fused_tp._ColumnParallelFused
                return fn.apply(x, self.weight, self.bias, self.reversed, activation is not None, tp)
        if mpu is not None:
            x = mpu.gather_sequence(x, dim=-2) if self.sequence_parallel else mpu.broadcast(x)
        if self.gather_output and mpu is not None and mpu.tp > 1:
            y = _linear(x, self.weight, None, self.reversed, self.oslo_fused)
            y = mpu.gather(y, dim=-1, full_size=self.full_out_features)
            if self.bias is not None:
                y = y + self.bias
            if activation is not None:
                y = ops.bias_gelu(y, None)
            return y
        return _linear(x, self.weight, self.bias, self.reversed, self.oslo_fused, activation)


class RowParallelLinear(nn.Linear):
    """Linear layer whose input features are split over the tensor-parallel group.

    forward: optional scatter -> GEMM -> all-reduce (or reduce-scatter along the sequence) -> bias.
    The bias is kept whole and added once, after the reduction (reference: oslo/modeling_utils.py:87-104).
    """

    oslo_fused = False
    mpu = None
    reversed = False
    input_is_parallel = True
    sequence_parallel = False

    def partial_forward(self, x: Tensor) -> Tensor:
        """This rank's partial sum ``x W^T`` without the reduction and without the bias; hand it to another
        row-parallel layer's ``forward(..., partial=...)`` so that both products share one collective."""
        if self.mpu is not None and not self.input_is_parallel:
            x = self.mpu.scatter(x, dim=-1)
        return _linear(x, self.weight, None, self.reversed, self.oslo_fused)

    def forward(self, x: Tensor, activation: Optional[str] = None, partial: Optional[Tensor] = None,
                residual: Optional[Tensor] = None) -> Tensor:
        """``partial``: partial sum of another row-parallel layer (``partial_forward``), reduced together with this
        layer's product; that layer's bias, if any, is the caller's business. ``residual`` (full tensor, same shape
        as the result) is added after the reduction, in the same pass as the bias on the kernel path."""
        mpu = self.mpu
        if mpu is not None and not self.input_is_parallel:
            x = mpu.scatter(x, dim=-1)
        if self.oslo_fused:
            from . import fused_tp
            n_out = self.weight.size(1) if self.reversed else self.weight.size(0)
            rows = x.numel() // max(x.size(-1), 1)
            if fused_tp.fused_tp_usable(mpu, x, n_out) and (not self.sequence_parallel or rows % (mpu.tp * 128) == 0):
                tp = fused_tp.get_fused_tp(mpu.get_tensor_parallel_group())
                if self.sequence_parallel:
                    from ..config import get_config
                    if partial is None or get_config().tp_shared_reduction_sp:
                        y = fused_tp._RowParallelSeqFused.apply(x, self.weight, self.reversed, tp, partial)
                    else:   # the shared form has not run on GPUs yet: keep the two reductions separate
                        y = fused_tp._RowParallelSeqFused.apply(x, self.weight, self.reversed, tp, None)
                        y = y + mpu.reduce_scatter_sequence(partial, dim=-2)
                else:
                    # with a bias the sum is consumed at once by the addition below, so the kernel's workspace slot
                    # is handed out as it is; without one the caller gets a tensor of its own
                    y = fused_tp._RowParallelFused.apply(x, self.weight, self.reversed, tp, partial,
                                                         self.bias is None and residual is None)
                if residual is not None and residual.shape == y.shape:
                    from ..ops import cuda_ops
                    return cuda_ops.bias_dropout_residual(y, self.bias, residual, 0.0, False)   # one pass over y
                y = y if self.bias is None else y + self.bias
                return y if residual is None else y + residual
        y = _linear(x, self.weight, None, self.reversed, self.oslo_fused)
        if partial is not None:
            y = y + partial
        if mpu is not None:
            y = mpu.reduce_scatter_sequence(y, dim=-2) if self.sequence_parallel else mpu.reduce(y)
        if self.bias is not None:
            y = y + self.bias
        return y if residual is None else y + residual
