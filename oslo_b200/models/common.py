"""Shared decoder-only transformer machinery for the GPT-2 / GPT-Neo / GPT-J families.

Each family supplies its modules under the HF parameter names; this file supplies the attention
core (eager library path and fused flash / decode-kernel path), the static KV cache, and the
six-function forward protocol (``preblock_fn -> block_fn(layer_id) -> postblock_fn -> head_fn ->
loss_fn -> organize_fn``; reference: oslo/parallelism_utils.py:71-131) that both the plain
``forward`` and the pipeline engine execute.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..modeling_utils import (BaseModelOutputWithPast, CausalLMOutputWithPast, PreTrainedModel,
                              SequenceClassifierOutputWithPast)


class StaticKVCache:
    """Pre-allocated key/value cache ``[layers][B, heads, T_max, D]`` written in place.

    Replaces the grow-by-``torch.cat`` cache of the reference (oslo/models/gptj/modeling_gptj.py:239-248):
    appends are slice writes, beam reordering is one ``index_select`` per tensor, and the decode
    attention kernel reads the first ``length`` positions.
    """

    def __init__(self, max_len: int) -> None:
        self.k: Dict[int, Tensor] = {}
        self.v: Dict[int, Tensor] = {}
        self.length = 0
        self.max_len = int(max_len)
        self.lengths_dev: Optional[Tensor] = None
        self.lengths_next: Optional[Tensor] = None
        # device-position mode (CUDA-graph decoding): single-token appends are index_copy_ at a position kept
        # in device memory, so the same captured step writes a new slot on every replay
        self.write_index: Optional[Tensor] = None
        self.device_positions = False

    def use_device_positions(self, on: bool = True) -> None:
        """Keep the write position of single-token appends on the device (needs one prior append). The position
        tensor is allocated once and updated in place, so a CUDA graph captured earlier keeps addressing it."""
        if not on:
            self.device_positions = False
            return
        if self.lengths_dev is None:
            raise RuntimeError("fill the cache (prefill) before switching to device positions")
        self.lengths_dev.fill_(self.length)
        self.lengths_next.fill_(self.length + 1)
        if self.write_index is None:
            self.write_index = torch.full((1,), self.length, dtype=torch.long, device=self.lengths_dev.device)
        else:
            self.write_index.fill_(self.length)
        self.device_positions = True

    def reset(self) -> None:
        """Forget the contents (storage is kept) so the cache can take a new prompt."""
        self.length = 0
        self.device_positions = False
        if self.lengths_dev is not None:
            self.lengths_dev.zero_()
            self.lengths_next.fill_(1)

    def append(self, layer: int, k: Tensor, v: Tensor) -> Tuple[Tensor, Tensor, int]:
        """Write ``k, v`` (``[B, heads, S, D]``) at the current position; returns the whole cache
        tensors of that layer and the new valid length. Storage is allocated on first use per layer."""
        b, h, s, d = k.shape
        if layer not in self.k:
            self.k[layer] = torch.zeros(b, h, self.max_len, d, dtype=k.dtype, device=k.device)
            self.v[layer] = torch.zeros(b, h, self.max_len, d, dtype=v.dtype, device=v.device)
        if self.lengths_dev is None:
            self.lengths_dev = torch.full((b,), self.length, dtype=torch.int32, device=k.device)
            self.lengths_next = self.lengths_dev + 1
        end = self.length + s
        if end > self.max_len:
            raise RuntimeError(f"KV cache overflow: {end} > {self.max_len}")
        if self.device_positions and s == 1:
            self.k[layer].index_copy_(2, self.write_index, k)
            self.v[layer].index_copy_(2, self.write_index, v)
            # `end` is only right outside graph replay; the decode kernel reads the valid length from lengths_next
            return self.k[layer], self.v[layer], end
        self.k[layer][:, :, self.length:end].copy_(k)
        self.v[layer][:, :, self.length:end].copy_(v)
        return self.k[layer], self.v[layer], end

    def advance(self, s: int) -> None:
        self.length += s
        self.lengths_dev.add_(s)
        self.lengths_next.add_(s)
        if self.device_positions:
            self.write_index.add_(s)

    def get_seq_length(self) -> int:
        return self.length

    def reorder(self, beam_idx: Tensor) -> "StaticKVCache":
        for i in list(self.k.keys()):
            self.k[i] = self.k[i].index_select(0, beam_idx)
            self.v[i] = self.v[i].index_select(0, beam_idx)
        if self.lengths_dev is not None and beam_idx.numel() != self.lengths_dev.numel():
            self.lengths_dev = self.lengths_dev[:1].expand(beam_idx.numel()).contiguous()
            self.lengths_next = self.lengths_next[:1].expand(beam_idx.numel()).contiguous()
        return self


def past_length(past_key_values) -> int:
    if past_key_values is None:
        return 0
    if isinstance(past_key_values, StaticKVCache):
        return past_key_values.get_seq_length()
    first = past_key_values[0]
    return 0 if first is None else first[0].size(-2)


class AttentionCore(nn.Module):
    """Softmax attention over ``[B, heads, S, D]`` with causal / local-window / padding masks.

    ``fused = False``: scores are materialised with library matmuls (the eager reference semantics).
    ``fused = True``: flash attention kernel for prefill / training, split-KV decode kernel for
    single-token steps on a static cache; ``output_attentions`` falls back to the fused softmax on
    materialised scores.
    """

    fused = False
    window: Optional[int] = None
    scale: float = 1.0
    attn_pdrop: float = 0.0

    def core_attention(self, q: Tensor, k: Tensor, v: Tensor, key_padding_mask: Optional[Tensor],
                       output_attentions: bool = False, head_mask: Optional[Tensor] = None,
                       cache_len: Optional[int] = None, lengths: Optional[Tensor] = None):
        """``k``/``v`` may be a whole static cache of which the first ``cache_len`` positions are valid."""
        p = self.attn_pdrop if self.training else 0.0
        if cache_len is not None and not (self.fused and q.size(2) == 1 and key_padding_mask is None
                                          and not output_attentions and head_mask is None):
            k, v = k[:, :, :cache_len], v[:, :, :cache_len]
            cache_len = None
        if cache_len is not None:
            out = ops.decode_attention(q[:, :, 0], k, v, lengths, self.scale, self.window)
            return out.unsqueeze(2), None
        if output_attentions or head_mask is not None or not self.fused:
            if self.fused and output_attentions and head_mask is None and p == 0.0:
                return self._fused_scores_attention(q, k, v, key_padding_mask)
            out, probs = ops.reference.attention(q, k, v, True, self.window, self.scale, key_padding_mask,
                                                 p, self.training, return_probs=True)
            if head_mask is not None:
                probs = probs * head_mask
                out = torch.matmul(probs, v.float()).to(q.dtype)
            return out, (probs.to(q.dtype) if output_attentions else None)
        out = ops.attention(q, k, v, True, self.window, self.scale, key_padding_mask, p, self.training)
        return out, None

    def _fused_scores_attention(self, q, k, v, key_padding_mask):
        from ..fused_kernels_utils import FusedScaleMaskSoftmax
        sq, sk = q.size(-2), k.size(-2)
        scores = torch.matmul(q, k.transpose(-1, -2))
        if sq == sk and self.window is None and key_padding_mask is None:
            probs = FusedScaleMaskSoftmax.apply(scores, None, self.scale, True)
        else:
            keep = ops.reference.attention_mask_bias(sq, sk, q.device, True, self.window)
            mask = ~keep[None, None]
            if key_padding_mask is not None:
                mask = mask | ~key_padding_mask.to(torch.bool)[:, None, None, :]
            probs = FusedScaleMaskSoftmax.apply(scores, mask.expand(q.size(0), 1, sq, sk), self.scale, False)
        return torch.matmul(probs, v), probs

    def attend_with_cache(self, q: Tensor, k: Tensor, v: Tensor, layer_past, cache: Optional[StaticKVCache],
                          layer_id: int, key_padding_mask, use_cache: bool, output_attentions: bool,
                          head_mask: Optional[Tensor]):
        """Handle both cache styles, then run ``core_attention``. Returns ``(out, present, probs)``."""
        if cache is not None:
            kc, vc, new_len = cache.append(layer_id, k, v)
            lengths = cache.lengths_next if q.size(2) == 1 else None
            out, probs = self.core_attention(q, kc, vc, key_padding_mask, output_attentions, head_mask,
                                             cache_len=new_len, lengths=lengths)
            return out, None, probs
        if layer_past is not None:
            k = torch.cat((layer_past[0], k), dim=-2)
            v = torch.cat((layer_past[1], v), dim=-2)
        present = (k, v) if use_cache else None
        out, probs = self.core_attention(q, k, v, key_padding_mask, output_attentions, head_mask)
        return out, present, probs


def split_heads(x: Tensor, num_heads: int, head_dim: int) -> Tensor:
    """``[B, S, heads*D] -> [B, heads, S, D]`` as a strided view (no copy)."""
    b, s, _ = x.shape
    return x.view(b, s, num_heads, head_dim).permute(0, 2, 1, 3)


def merge_heads(x: Tensor) -> Tensor:
    """``[B, heads, S, D] -> [B, S, heads*D]``."""
    b, h, s, d = x.shape
    return x.permute(0, 2, 1, 3).reshape(b, s, h * d)


def to_batch_seq(x: Tensor, seq_shape) -> Tensor:
    """``[1, B*S, n] -> [B, S, n]`` under sequence parallelism (identity otherwise)."""
    return x if seq_shape is None else x.reshape(seq_shape[0], seq_shape[1], x.size(-1))


def to_token_rows(x: Tensor, seq_shape) -> Tensor:
    """``[B, S, n] -> [1, B*S, n]`` under sequence parallelism (identity otherwise)."""
    return x if seq_shape is None else x.reshape(1, seq_shape[0] * seq_shape[1], x.size(-1))


def maybe_dropout(x: Tensor, p: float, training: bool) -> Tensor:
    return F.dropout(x, p, training) if (p > 0.0 and training) else x


class DecoderBackbone(PreTrainedModel):
    """Base of ``GPT2Model`` / ``GPTNeoModel`` / ``GPTJModel``: embeddings, ``h`` blocks, ``ln_f``."""

    def embed(self, input_ids, position_ids, token_type_ids, inputs_embeds) -> Tensor:
        raise NotImplementedError

    def get_input_embeddings(self):
        return self.wte

    def set_input_embeddings(self, value):
        self.wte = value

    def num_blocks(self) -> int:
        return len(self.h)

    # ------------------------------------------------------------------ protocol
    def prepare_fn(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None,
                   position_ids=None, head_mask=None, inputs_embeds=None, use_cache=None,
                   output_attentions=None, output_hidden_states=None, return_dict=None, **rest) -> Dict[str, Any]:
        """Parameter-free input normalisation; every pipeline stage runs it on its own copy of the batch."""
        cfg = self.config
        output_attentions = cfg.output_attentions if output_attentions is None else output_attentions
        output_hidden_states = cfg.output_hidden_states if output_hidden_states is None else output_hidden_states
        use_cache = cfg.use_cache if use_cache is None else use_cache
        return_dict = cfg.return_dict if return_dict is None else return_dict
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("pass either input_ids or inputs_embeds, not both")
        if input_ids is not None:
            input_ids = input_ids.view(-1, input_ids.size(-1))
            bsz, seq = input_ids.shape
            device = input_ids.device
        elif inputs_embeds is not None:
            bsz, seq = inputs_embeds.shape[:2]
            device = inputs_embeds.device
        elif rest.get("hidden_states") is not None:
            bsz, seq = rest["hidden_states"].shape[:2]
            device = rest["hidden_states"].device
        else:
            raise ValueError("input_ids or inputs_embeds is required")
        cache = past_key_values if isinstance(past_key_values, StaticKVCache) else None
        past_len = past_length(past_key_values)
        if cache is not None or past_key_values is None:
            layer_pasts = [None] * self.num_blocks()
        else:
            layer_pasts = list(past_key_values)
        if position_ids is None:
            position_ids = torch.arange(past_len, past_len + seq, dtype=torch.long, device=device)
            position_ids = position_ids.unsqueeze(0).expand(bsz, seq)
        else:
            position_ids = position_ids.view(-1, seq)
        if token_type_ids is not None:
            token_type_ids = token_type_ids.view(-1, seq)
        if attention_mask is not None:
            attention_mask = attention_mask.view(bsz, -1)
            if bool((attention_mask != 0).all()) if attention_mask.device.type == "cpu" else False:
                attention_mask = None
        if head_mask is not None and head_mask.dim() == 1:
            head_mask = head_mask[None, :].expand(self.num_blocks(), -1)
        out = dict(rest)
        if self.sequence_parallel_active():
            # a training layout: no KV cache, and the token rows must split evenly over the group
            if (bsz * seq) % (self.mpu.tp) or past_len:
                raise ValueError("sequence parallelism needs batch*seq divisible by tensor_parallel_size and no past")
            use_cache, cache, layer_pasts = False, None, [None] * self.num_blocks()
            out_bs = (bsz, seq)
        else:
            out_bs = None
        out.update(
            _bs=out_bs, input_ids=input_ids, inputs_embeds=inputs_embeds, token_type_ids=token_type_ids,
            position_ids=position_ids, attention_mask=attention_mask, head_mask=head_mask,
            layer_pasts=layer_pasts, cache=cache, use_cache=use_cache, output_attentions=output_attentions,
            output_hidden_states=output_hidden_states, return_dict=return_dict,
            presents=[] if (use_cache and cache is None) else None,
            all_hidden_states=[] if output_hidden_states else None,
            all_attentions=[] if output_attentions else None, _seq=seq,
        )
        return out

    def sequence_parallel_active(self) -> bool:
        mpu = getattr(self, "mpu", None)
        return bool(getattr(self, "sequence_parallel", False)) and mpu is not None and mpu.tp > 1

    def preblock_fn(self, **kw) -> Dict[str, Any]:
        kw = self.prepare_fn(**kw)
        hs = self.embed(kw["input_ids"], kw["position_ids"], kw["token_type_ids"], kw["inputs_embeds"])
        if self.sequence_parallel_active():
            # sequence parallelism: between the tensor-parallel GEMMs every rank keeps 1/tp of the flattened
            # (batch, position) token rows; the column-parallel layers gather them, the row-parallel ones scatter
            b, s_, h = hs.shape
            hs = self.mpu.scatter(hs.reshape(1, b * s_, h), dim=1)
        kw["hidden_states"] = hs
        return kw

    def block_fn(self, layer_id: int, **kw) -> Dict[str, Any]:
        block = self.h[layer_id]
        hs = kw["hidden_states"]
        if kw["all_hidden_states"] is not None:
            kw["all_hidden_states"].append(hs)
        hm = kw["head_mask"][layer_id].view(1, -1, 1, 1) if kw["head_mask"] is not None else None
        args = dict(layer_past=kw["layer_pasts"][layer_id], attention_mask=kw["attention_mask"],
                    position_ids=kw["position_ids"], head_mask=hm, use_cache=kw["use_cache"],
                    output_attentions=kw["output_attentions"], cache=kw["cache"], layer_id=layer_id)
        if kw.get("_bs") is not None:
            args["seq_shape"] = kw["_bs"]
        for extra in ("encoder_hidden_states", "encoder_attention_mask"):
            if kw.get(extra) is not None:
                args[extra] = kw[extra]
        if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
            args["use_cache"] = False
            hs, present, probs = checkpoint(lambda h: block(h, **args), hs, use_reentrant=False)
        else:
            hs, present, probs = block(hs, **args)
        kw["hidden_states"] = hs
        if kw["presents"] is not None:
            kw["presents"].append(present)
        if kw["all_attentions"] is not None:
            kw["all_attentions"].append(probs)
        return kw

    def postblock_fn(self, **kw) -> Dict[str, Any]:
        hs = self.ln_f(kw["hidden_states"])
        if kw.get("_bs") is not None:
            b, s_ = kw["_bs"]
            # what follows (head, loss) is computed identically on every rank and its input gradient is already
            # summed over the group, so the backward of this gather keeps the local rows (no second reduction)
            hs = self.mpu.gather(hs, dim=1, full_size=b * s_).reshape(b, s_, hs.size(-1))
        if kw["all_hidden_states"] is not None:
            kw["all_hidden_states"].append(hs)
        if kw["cache"] is not None:
            kw["cache"].advance(kw["_seq"])
        kw["hidden_states"] = hs
        return kw

    def collect_past(self, kw):
        if kw.get("cache") is not None:
            return kw["cache"]
        return tuple(kw["presents"]) if kw.get("presents") else None

    def organize_fn(self, **kw):
        out = BaseModelOutputWithPast(
            last_hidden_state=kw["hidden_states"], past_key_values=self.collect_past(kw),
            hidden_states=tuple(kw["all_hidden_states"]) if kw["all_hidden_states"] is not None else None,
            attentions=tuple(kw["all_attentions"]) if kw["all_attentions"] is not None else None)
        return out if kw["return_dict"] else out.to_tuple()

    def forward(self, input_ids=None, **kw):
        return self.run_protocol(input_ids=input_ids, **kw)


def run_forward_pre_hooks(module: nn.Module) -> None:
    """Run ``module``'s forward pre-hooks without calling it. Code that reads a module's parameters directly (the LM
    head's weight handed to the fused loss) calls this first: wrappers hang per-module work on those hooks - the
    data-parallel wrapper makes the compute stream wait there for the parameter buckets that are still in flight
    after the optimizer step - and they must see every use of the parameters, not only ``module(...)`` calls."""
    with_kwargs = getattr(module, "_forward_pre_hooks_with_kwargs", {})
    for hid, hook in list(module._forward_pre_hooks.items()):
        if with_kwargs.get(hid):
            hook(module, (), {})
        else:
            hook(module, ())


def shifted_lm_labels(labels: Tensor) -> Tensor:
    """Labels aligned with logits rows: position ``i`` predicts token ``i+1``; the last column is ignored."""
    shifted = torch.full_like(labels, -100)
    shifted[..., :-1] = labels[..., 1:]
    return shifted


class CausalLMHeadMixin:
    """``head_fn`` / ``loss_fn`` / ``organize_fn`` of an LM-head model (``self.lm_head`` over ``self.transformer``).

    With ``output_logits=False`` and labels given, the projection and the loss run as one fused,
    row-chunked op so the ``[tokens, vocab]`` logits never exist; under tensor parallelism a
    vocabulary-sharded head computes the loss from shard-local statistics (max, sum-exp, target
    logit) combined by all-reduces instead of all-gathering logits as the reference does
    (oslo/parallelism/mpu.py:759).
    """

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new):
        self.lm_head = new

    def num_blocks(self) -> int:
        return self.transformer.num_blocks()

    def head_fn(self, **kw):
        hs = kw["hidden_states"]
        labels = kw.get("labels")
        head = self.lm_head
        mpu = getattr(head, "mpu", None)
        want_logits = kw.get("output_logits", True) or labels is None
        if kw.get("last_token_logits") and labels is None:
            hs = hs[:, -1:, :]
        kw["logits"] = None
        kw["loss"] = None
        vocab_sharded = mpu is not None and mpu.tp > 1 and getattr(head, "vocab_parallel", False)
        if vocab_sharded or not want_logits:
            run_forward_pre_hooks(head)      # the branches below read head.weight / head.bias without calling head
        if want_logits:
            if vocab_sharded:
                x = mpu.broadcast(hs)
                local = ops.linear(x, head.weight, head.bias) if head.oslo_fused else F.linear(x, head.weight, head.bias)
                kw["logits"] = mpu.gather(local, dim=-1, full_size=head.full_out_features)
            else:
                kw["logits"] = head(hs)
            return kw
        tgt = shifted_lm_labels(labels).reshape(-1)
        flat = hs.reshape(-1, hs.size(-1))
        if vocab_sharded:
            from ..parallel.vocab_parallel import vocab_parallel_linear_cross_entropy
            kw["loss"] = vocab_parallel_linear_cross_entropy(flat, head.weight, head.bias, tgt, mpu,
                                                             head.full_out_features, fused=head.oslo_fused)
        elif head.oslo_fused:
            kw["loss"] = ops.linear_cross_entropy(flat, head.weight, head.bias, tgt)
        else:
            kw["loss"] = ops.reference.cross_entropy(F.linear(flat, head.weight, head.bias), tgt)
        return kw

    def loss_fn(self, **kw):
        labels = kw.get("labels")
        if labels is not None and kw.get("loss") is None:
            logits = kw["logits"]
            shift = logits[..., :-1, :].contiguous()
            tgt = labels[..., 1:].contiguous().view(-1)
            flat = shift.view(-1, shift.size(-1))
            fused = getattr(self.lm_head, "oslo_fused", False)
            kw["loss"] = ops.cross_entropy(flat, tgt) if fused else ops.reference.cross_entropy(flat, tgt)
        return kw

    def organize_fn(self, **kw):
        base = self.transformer
        out = CausalLMOutputWithPast(
            loss=kw.get("loss"), logits=kw.get("logits"), past_key_values=base.collect_past(kw),
            hidden_states=tuple(kw["all_hidden_states"]) if kw["all_hidden_states"] is not None else None,
            attentions=tuple(kw["all_attentions"]) if kw["all_attentions"] is not None else None)
        return out if kw["return_dict"] else out.to_tuple()

    def forward(self, input_ids=None, **kw):
        return self.run_protocol(input_ids=input_ids, **kw)

    # ------------------------------------------------------------------ generation hooks
    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kwargs):
        position_ids = kwargs.get("position_ids")
        if attention_mask is not None and position_ids is None:
            position_ids = attention_mask.long().cumsum(-1) - 1
            position_ids.masked_fill_(attention_mask == 0, 1)
        if past_length(past_key_values) > 0:
            input_ids = input_ids[:, -1:]
            if position_ids is not None:
                position_ids = position_ids[:, -1:]
        if attention_mask is not None and bool((attention_mask != 0).all()):
            attention_mask = None
        return dict(input_ids=input_ids, past_key_values=past_key_values, use_cache=kwargs.get("use_cache", True),
                    position_ids=position_ids, attention_mask=attention_mask,
                    token_type_ids=None)

    @staticmethod
    def _reorder_cache(past, beam_idx: Tensor):
        if isinstance(past, StaticKVCache):
            return past.reorder(beam_idx)
        return tuple(tuple(t.index_select(0, beam_idx.to(t.device)) for t in layer) for layer in past)


class SequenceClassificationMixin:
    """Classification from the hidden state of the last non-pad token (``self.score`` over ``self.transformer``)."""

    def num_blocks(self) -> int:
        return self.transformer.num_blocks()

    def head_fn(self, **kw):
        kw["logits_all"] = self.score(kw["hidden_states"])
        return kw

    def loss_fn(self, **kw):
        logits_all = kw["logits_all"]
        input_ids = kw.get("input_ids")
        bsz = logits_all.size(0)
        pad = self.config.pad_token_id
        if pad is None or input_ids is None:
            if bsz != 1 and pad is None:
                raise ValueError("batch sizes > 1 need config.pad_token_id")
            last = torch.full((bsz,), -1, device=logits_all.device, dtype=torch.long)
        else:
            last = (torch.ne(input_ids, pad).sum(-1) - 1).to(logits_all.device)
        pooled = logits_all[torch.arange(bsz, device=logits_all.device), last]
        kw["logits"] = pooled
        labels = kw.get("labels")
        kw["loss"] = None
        if labels is not None:
            n = self.num_labels
            if n == 1:
                kw["loss"] = F.mse_loss(pooled.view(-1).float(), labels.view(-1).float())
            elif labels.dtype in (torch.long, torch.int):
                kw["loss"] = F.cross_entropy(pooled.view(-1, n).float(), labels.view(-1))
            else:
                kw["loss"] = F.binary_cross_entropy_with_logits(pooled.float(), labels.float())
        return kw

    def organize_fn(self, **kw):
        base = self.transformer
        out = SequenceClassifierOutputWithPast(
            loss=kw.get("loss"), logits=kw.get("logits"), past_key_values=base.collect_past(kw),
            hidden_states=tuple(kw["all_hidden_states"]) if kw["all_hidden_states"] is not None else None,
            attentions=tuple(kw["all_attentions"]) if kw["all_attentions"] is not None else None)
        return out if kw["return_dict"] else out.to_tuple()

    def forward(self, input_ids=None, **kw):
        return self.run_protocol(input_ids=input_ids, **kw)
