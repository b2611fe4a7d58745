"""Tensor-parallel engine: policy-driven in-place weight slicing, and the inverse merge.

Behaviour contract (reference: oslo/parallelism/engine_tensor.py:44-460, :463-819):

* column-parallel layers are cut along the output features (+ bias), row-parallel layers along the
  input features (bias kept whole);
* a fused projection (``n_fused`` = 3 for GPT-2's ``c_attn``) is cut into ``n_fused * tp`` pieces and
  rank ``r`` keeps pieces ``r, r + tp, r + 2 tp`` so its shard reads ``[q_r | k_r | v_r]``;
* embedding rows are cut with ``torch.chunk`` (ceil-sized, last shard short);
* ``reversed`` flips the cut axis for the ``[in, out]`` Conv1D layout;
* the module class is swapped afterwards, parameter names never change.

How every parameter was cut is recorded in ``model._tp_specs`` so the merge needs no second model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .layers import (ColumnParallelLinear, Conv1D, Embedding, Linear, RowParallelLinear,
                     VocabParallelEmbedding)
from .mpu import MPU, Layer, ceil_split_sizes


class VocabParallelHead(ColumnParallelLinear):
    """LM head whose weight rows are a vocabulary shard (tied to a ``VocabParallelEmbedding`` or own)."""

    vocab_parallel = True


@dataclass
class ShardSpec:
    kind: str          # "column" | "row" | "vocab"
    dim: int           # axis that was cut
    n_fused: int
    full_size: int     # size of that axis before the cut


def _chunk_ceil(t: Tensor, parts: int, dim: int) -> List[Tensor]:
    sizes = ceil_split_sizes(t.size(dim), parts)
    return list(torch.split(t, sizes, dim=dim))


def shard_tensor(t: Tensor, tp: int, rank: int, dim: int, n_fused: int = 1) -> Tensor:
    """This rank's shard of ``t`` along ``dim`` (fused tensors are regrouped per rank)."""
    if n_fused > 1:
        if t.size(dim) % (n_fused * tp):
            raise ValueError(f"axis {dim} of size {t.size(dim)} is not divisible by n_fused*tp={n_fused * tp}")
        pieces = torch.chunk(t, n_fused * tp, dim=dim)
        return torch.cat([pieces[rank + i * tp] for i in range(n_fused)], dim=dim).clone()
    return _chunk_ceil(t, tp, dim)[rank].clone()


def unshard_tensors(shards: List[Tensor], dim: int, n_fused: int = 1) -> Tensor:
    """Inverse of ``shard_tensor`` given every rank's shard in rank order."""
    if n_fused > 1:
        per_rank = [torch.chunk(s, n_fused, dim=dim) for s in shards]
        ordered = [per_rank[r][i] for i in range(n_fused) for r in range(len(shards))]
        return torch.cat(ordered, dim=dim)
    return torch.cat(shards, dim=dim)


class TensorParallelEngine:
    def __init__(self, model: nn.Module, mpu: MPU, owned: Optional[Callable[[Tensor], bool]] = None,
                 device=None, sequence_parallel: bool = False) -> None:
        self.model, self.mpu = model, mpu
        # ``owned(param)``: does this rank's pipeline stage hold the parameter (tied weights may be
        # held by a stage that does not own the module they are declared in)
        self.owned = owned or (lambda p: True)
        self.device = device
        self.sequence_parallel = sequence_parallel
        self.tp, self.rank = mpu.get_tensor_parallel_world_size(), mpu.get_tensor_parallel_rank()
        self._names = {}
        for n, p in model.named_parameters(remove_duplicate=False):
            self._names.setdefault(id(p), []).append(n)
        self.specs: Dict[str, ShardSpec] = {}
        self._sp_partial: List[Optional[nn.Parameter]] = []
        self._in_block_or_post = False

    # ------------------------------------------------------------------ public
    def parallelize(self) -> None:
        model, cfg = self.model, self.model.config
        for policy in model.get_layer_policies():
            for layer in policy.word_embedding(model, cfg):
                self._vocab(layer)
            for layer in policy.preblock_layers(model, cfg):
                self._replicated(layer)
            for block in policy.block_layers(model, cfg):
                self._block(policy, block, cfg)
            for layer in policy.postblock_layers(model, cfg):
                self._replicated(layer)
                self._sp_partial += [layer.weight, layer.bias]
        for layer in model.get_head_layers():
            self._head(layer)
        model._tp_specs = self.specs
        # parameters that were not cut exist once per tensor-parallel rank with the same gradient: in a global
        # gradient norm only the copy on rank 0 counts (FusedAdamW.grad_norm leaves the marked ones out)
        if self.rank != 0:
            for p in model.parameters():
                if not getattr(p, "_oslo_tp_sharded", False):
                    p._oslo_norm_dup = True
        if self.sequence_parallel:
            model.base_model.sequence_parallel = True
            # parameters applied to a token shard see only 1/tp of the tokens: their gradients are partial sums
            model._sp_partial_params = [p for p in self._sp_partial if p is not None]

    # ------------------------------------------------------------------ pieces
    def _block(self, policy, block: nn.Module, cfg) -> None:
        heads = getattr(cfg, "n_head", None) or getattr(cfg, "num_heads", None)
        hidden = getattr(cfg, "n_embd", None) or getattr(cfg, "hidden_size", None)
        if heads is not None and (heads < self.tp or heads % self.tp):
            raise ValueError(f"attention heads ({heads}) must be a multiple of tensor_parallel_size ({self.tp})")
        if hidden is not None and hidden < self.tp:
            raise ValueError(f"hidden size ({hidden}) is smaller than tensor_parallel_size ({self.tp})")
        policy.reduce_arguments(block, self.tp, cfg)
        for layer in policy.attn_qkv(block, cfg) + policy.mlp_in(block, cfg):
            self._column(layer)
        for layer in policy.attn_out(block, cfg) + policy.mlp_out(block, cfg):
            self._row(layer)
        for layer in policy.attn_norm(block, cfg) + policy.mlp_norm(block, cfg) + policy.copy_to_all(block, cfg):
            self._replicated(layer)
            self._sp_partial += [layer.weight, layer.bias]

    def _record(self, p: Tensor, spec: ShardSpec) -> None:
        for n in self._names.get(id(p), []):
            self.specs[n] = spec

    def _cut(self, p: Optional[nn.Parameter], dim: int, n_fused: int, kind: str, module: nn.Module) -> None:
        if p is None:
            return
        self._record(p, ShardSpec(kind, dim, n_fused, p.size(dim) if p.numel() else -1))
        p._oslo_tp_sharded = True
        if self.owned(p) and p.numel():
            p.data = shard_tensor(p.data, self.tp, self.rank, dim, n_fused)

    def _column(self, layer: Layer) -> None:
        m = layer.module
        wdim = 1 if layer.reversed else 0
        full_out = layer.weight.size(wdim)
        self._cut(layer.weight, wdim, layer.n_fused, "column", m)
        self._cut(layer.bias, 0, layer.n_fused, "column", m)
        self._swap(m, ColumnParallelLinear, layer)
        m.gather_output = layer.gather_output
        m.full_out_features = full_out
        m.sequence_parallel = self.sequence_parallel
        self._set_features(m, layer)

    def _row(self, layer: Layer) -> None:
        m = layer.module
        wdim = 0 if layer.reversed else 1
        self._cut(layer.weight, wdim, layer.n_fused, "row", m)
        if layer.bias is not None:
            self._record(layer.bias, ShardSpec("replicated", 0, 1, layer.bias.size(0)))
            self._sp_partial.append(layer.bias)
        self._swap(m, RowParallelLinear, layer)
        m.input_is_parallel = layer.input_is_parallel
        m.sequence_parallel = self.sequence_parallel
        self._set_features(m, layer)

    def _vocab(self, layer: Layer) -> None:
        m = layer.module
        full = layer.weight.size(0)
        self._cut(layer.weight, 0, 1, "vocab", m)
        m.__class__ = VocabParallelEmbedding
        m.mpu = self.mpu
        m.full_num_embeddings = full
        m.num_embeddings = ceil_split_sizes(full, self.tp)[self.rank]

    def _head(self, layer: Layer) -> None:
        m = layer.module
        if layer.replace and "vocab_head" in layer.replace.values():
            if layer.tied_embedding is not None:
                full = layer.tied_embedding.full_num_embeddings
            else:
                full = layer.weight.size(0)
                self._cut(layer.weight, 0, 1, "vocab", m)
                self._cut(layer.bias, 0, 1, "vocab", m)
            self._swap(m, VocabParallelHead, layer)
            m.gather_output = True
            m.full_out_features = full
            m.out_features = ceil_split_sizes(full, self.tp)[self.rank]
            return
        self._replicated(layer)

    def _replicated(self, layer: Layer) -> None:
        for p in (layer.weight, layer.bias):
            if p is not None:
                self._record(p, ShardSpec("replicated", 0, 1, p.size(0) if p.dim() else 1))
        if layer.module is not None and hasattr(type(layer.module), "mpu"):
            layer.module.mpu = self.mpu

    def _swap(self, m: nn.Module, cls: type, layer: Layer) -> None:
        m.__class__ = cls
        m.mpu = self.mpu
        m.reversed = layer.reversed

    @staticmethod
    def _set_features(m: nn.Module, layer: Layer) -> None:
        w = layer.weight
        if w.numel():
            m.in_features = w.size(0) if layer.reversed else w.size(1)
            m.out_features = w.size(1) if layer.reversed else w.size(0)


class TensorDeparallelEngine:
    """Rebuild whole tensors from tensor-parallel shards (all-gather per parameter, cold path)."""

    def __init__(self, model: nn.Module, mpu: MPU) -> None:
        self.model, self.mpu = model, mpu
        self.specs: Dict[str, ShardSpec] = getattr(model, "_tp_specs", {})

    def merge_state(self, state: Dict[str, Tensor]) -> Dict[str, Tensor]:
        """Merged CPU state dict. Every rank of the TP group must call this with the same keys."""
        tp = self.mpu.get_tensor_parallel_world_size()
        out: Dict[str, Tensor] = {}
        for name in sorted(state.keys()):
            t = state[name]
            spec = self.specs.get(name)
            if tp == 1 or spec is None or spec.kind == "replicated":
                out[name] = t.detach().cpu()
                continue
            shards = self._all_gather_shards(t.detach(), spec)
            out[name] = unshard_tensors(shards, spec.dim, spec.n_fused).cpu()
        return out

    def _all_gather_shards(self, t: Tensor, spec: ShardSpec) -> List[Tensor]:
        mpu = self.mpu
        tp = mpu.get_tensor_parallel_world_size()
        dev = mpu.device
        t = t.to(dev)
        if spec.n_fused > 1:
            sizes = [t.size(spec.dim)] * tp
        else:
            sizes = ceil_split_sizes(spec.full_size, tp)
        big = max(sizes)
        if t.size(spec.dim) != big:
            pad = list(t.shape)
            pad[spec.dim] = big - t.size(spec.dim)
            t = torch.cat([t, t.new_zeros(pad)], dim=spec.dim)
        t = t.contiguous()
        bufs = [torch.empty_like(t) for _ in range(tp)]
        dist.all_gather(bufs, t, group=mpu.get_tensor_parallel_group())
        return [b.narrow(spec.dim, 0, s).cpu() for b, s in zip(bufs, sizes)]

    def deparallelize(self) -> nn.Module:
        """Turn the live model back into a single-device model (weights merged, classes restored)."""
        merged = self.merge_state(self.model.state_dict())
        restore = {ColumnParallelLinear: None, RowParallelLinear: None}
        for m in self.model.modules():
            cls = type(m)
            if cls in (ColumnParallelLinear, RowParallelLinear) or cls.__name__ == "VocabParallelHead":
                m.__class__ = Conv1D if getattr(m, "reversed", False) else Linear
                m.__dict__.pop("mpu", None)
            elif cls is VocabParallelEmbedding:
                m.__class__ = Embedding
                m.__dict__.pop("mpu", None)
                m.num_embeddings = m.full_num_embeddings
        named = dict(self.model.named_parameters(remove_duplicate=False))
        for name, t in merged.items():
            if name in named:
                named[name].data = t.to(named[name].dtype)
        for m in self.model.modules():
            if isinstance(m, (Linear,)) and not isinstance(m, (ColumnParallelLinear, RowParallelLinear)):
                m.out_features, m.in_features = m.weight.shape
        cfg = self.model.config
        for policy in self.model.get_layer_policies():
            for block in policy.block_layers(self.model, cfg):
                policy.reduce_arguments(block, 1, cfg)
        self.model._tp_specs = {}
        return self.model
