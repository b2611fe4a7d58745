"""GPT-J: parallel attention+MLP residual, interleaved rotary embedding on the first ``rotary_dim`` dims.

Semantics follow the eager model of the reference (oslo/models/gptj/modeling_gptj.py: block
:306-320, rotary :49-77, attention :151-191, loss :749-768) with the fused-path scale bug fixed:
scores are always multiplied by ``1/sqrt(head_dim)``.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from ...config import get_config
from ...fused_kernels_utils import ACT2FN, GELU_TANH_NAMES
from ...modeling_utils import PretrainedConfig, PreTrainedModel
from ...parallel.layers import Embedding, LayerNorm, Linear, RowParallelLinear
from ...parallel.mpu import Layer, LayerPolicy
from ..common import (AttentionCore, CausalLMHeadMixin, DecoderBackbone, SequenceClassificationMixin,
                      maybe_dropout, merge_heads, to_token_rows)


def fixed_pos_embedding(x: Tensor, seq_dim: int = 1, seq_len: Optional[int] = None):
    """``(sin, cos)`` tables ``[seq_len, x.shape[-1] // 2]`` for positions ``0 .. seq_len - 1`` (fp32, on ``x``'s device).
    The three rotary helpers below keep the names and call conventions of the reference's module-level functions
    (oslo/models/gptj/modeling_gptj.py:49-77) for code that imports them; the model itself goes through
    ``ops.rotary_interleaved`` (one kernel on GPUs)."""
    n = x.shape[seq_dim] if seq_len is None else int(seq_len)
    return ops.reference.rotary_tables(torch.arange(n, device=x.device), x.shape[-1])


def rotate_every_two(x: Tensor) -> Tensor:
    """``(x0, x1, x2, x3, ...) -> (-x1, x0, -x3, x2, ...)`` along the last dimension."""
    pairs = x.unflatten(-1, (-1, 2))
    return torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).flatten(-2)


def apply_rotary_pos_emb(x: Tensor, sincos, offset: int = 0) -> Tensor:
    """Rotate ``x`` ``[batch, seq, heads, dim]`` by the table rows ``offset .. offset + seq`` (each sin / cos value
    serves one pair of neighbouring dimensions)."""
    sin, cos = (t[offset: offset + x.shape[1]].repeat_interleave(2, dim=-1)[None, :, None, :] for t in sincos)
    return x * cos + rotate_every_two(x) * sin


class GPTJConfig(PretrainedConfig):
    model_type = "gptj"
    attribute_map = {"max_position_embeddings": "n_positions", "hidden_size": "n_embd",
                     "num_attention_heads": "n_head", "num_hidden_layers": "n_layer"}

    def __init__(self, vocab_size=50400, n_positions=2048, n_embd=4096, n_layer=28, n_head=16, rotary_dim=64,
                 n_inner=None, activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                 layer_norm_epsilon=1e-5, initializer_range=0.02, scale_attn_weights=True, use_cache=True,
                 bos_token_id=50256, eos_token_id=50256, tie_word_embeddings=False, **kwargs):
        self.vocab_size, self.n_positions, self.n_embd, self.n_layer, self.n_head = vocab_size, n_positions, n_embd, n_layer, n_head
        self.n_inner, self.rotary_dim, self.activation_function = n_inner, rotary_dim, activation_function
        self.resid_pdrop, self.embd_pdrop, self.attn_pdrop = resid_pdrop, embd_pdrop, attn_pdrop
        self.layer_norm_epsilon, self.initializer_range, self.scale_attn_weights = layer_norm_epsilon, initializer_range, scale_attn_weights
        super().__init__(use_cache=use_cache, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kwargs)


class GPTJAttention(AttentionCore):
    def __init__(self, config: GPTJConfig) -> None:
        super().__init__()
        self.embed_dim = config.n_embd
        self.num_attention_heads = config.n_head
        self.head_dim = self.embed_dim // self.num_attention_heads
        if self.head_dim * self.num_attention_heads != self.embed_dim:
            raise ValueError("n_embd must be divisible by n_head")
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.rotary_dim = config.rotary_dim
        self.attn_pdrop, self.resid_pdrop = config.attn_pdrop, config.resid_pdrop
        self.k_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.v_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.q_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.out_proj = Linear(self.embed_dim, self.embed_dim, bias=False)

    def forward(self, hidden_states: Tensor, layer_past=None, attention_mask=None, position_ids=None,
                head_mask=None, use_cache=False, output_attentions=False, cache=None, layer_id=0, seq_shape=None,
                qkv=None, residual=None, partial_only=False):
        b, s = seq_shape if seq_shape is not None else hidden_states.shape[:2]
        nh, hd = self.num_attention_heads, self.head_dim
        if qkv is not None:   # already projected by the block's packed decode GEMM
            q, k, v = (t.reshape(b, s, nh, hd) for t in qkv)
        elif self._one_node_qkv(hidden_states):
            from ...ops import cuda_ops
            q, k, v = (t.view(b, s, nh, hd) for t in cuda_ops.qkv_linear(
                hidden_states, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight))
        else:
            q = self.q_proj(hidden_states).view(b, s, nh, hd)
            k = self.k_proj(hidden_states).view(b, s, nh, hd)
            v = self.v_proj(hidden_states).view(b, s, nh, hd)
        rd = self.rotary_dim if self.rotary_dim is not None else hd
        rot = ops.rotary_interleaved if self.fused else ops.reference.rotary_interleaved
        q, k = rot(q, position_ids, rd), rot(k, position_ids, rd)
        q, k, v = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        out, present, probs = self.attend_with_cache(q, k, v, layer_past, cache, layer_id, attention_mask,
                                                     use_cache, output_attentions, head_mask)
        merged = to_token_rows(merge_heads(out), seq_shape)
        if partial_only:   # tensor parallel: leave the reduction to fc_out, which adds this partial sum to its own
            return self.out_proj.partial_forward(merged), present, probs
        if residual is not None:   # only offered by the block when out_proj is a plain Linear and no dropout follows
            return self.out_proj(merged, residual=residual), present, probs
        out = self.out_proj(merged)
        return maybe_dropout(out, self.resid_pdrop, self.training), present, probs

    def _one_node_qkv(self, x: Tensor) -> bool:
        """q, k, v as one autograd node (their input gradients accumulate inside the GEMM epilogues): plain fused
        bias-free ``Linear`` layers on a CUDA input that takes the large-input GEMM path."""
        layers = (self.q_proj, self.k_proj, self.v_proj)
        if not (self.fused and x.is_cuda and all(type(l) is Linear and l.oslo_fused and l.bias is None for l in layers)):
            return False
        if not get_config().block_fusion:
            return False
        from ...ops import cuda_ops
        return cuda_ops.qkv_linear_ok(x, *(l.weight for l in layers))


class FusedGPTJAttention(GPTJAttention):
    fused = True


class GPTJMLP(nn.Module):
    fused = False

    def __init__(self, intermediate_size: int, config: GPTJConfig) -> None:
        super().__init__()
        self.fc_in = Linear(config.n_embd, intermediate_size)
        self.fc_out = Linear(intermediate_size, config.n_embd)
        self.activation = config.activation_function
        self.resid_pdrop = config.resid_pdrop

    def forward(self, x: Tensor, h: Optional[Tensor] = None, residual: Optional[Tensor] = None,
                partial: Optional[Tensor] = None) -> Tensor:
        """``residual`` (only passed when no dropout follows) is added to the result, inside fc_out's GEMM epilogue
        where the fused path applies. ``partial`` (tensor parallel, no dropout): the attention output projection's
        partial sum, reduced together with fc_out's."""
        if partial is not None:
            if h is not None:
                act = h
            elif self.fused and self.activation in GELU_TANH_NAMES:
                act = self.fc_in(x, activation="gelu_new")
            else:
                act = ACT2FN[self.activation](self.fc_in(x))
            return self.fc_out(act, partial=partial, residual=residual)
        if residual is not None:
            return self._forward(x, h, residual)
        return self._forward(x, h, None)

    def _forward(self, x: Tensor, h: Optional[Tensor], residual: Optional[Tensor]) -> Tensor:
        if h is not None:     # fc_in + GeLU already done by the block's packed decode GEMM
            pass
        elif (self.fused and self.activation in GELU_TANH_NAMES and type(self.fc_in) is Linear
              and type(self.fc_out) is Linear and x.is_cuda and self.fc_in.oslo_fused and self.fc_out.oslo_fused):
            from ...ops import cuda_ops
            if cuda_ops.fused_mlp_ok(x, self.fc_in.weight, self.fc_out.weight):   # both layers in one autograd node
                y = cuda_ops.fused_mlp(x, self.fc_in.weight, self.fc_in.bias, self.fc_out.weight, self.fc_out.bias,
                                       residual)
                return y if residual is not None else maybe_dropout(y, self.resid_pdrop, self.training)
            h = self.fc_in(x, activation="gelu_new")
        elif self.fused and self.activation in GELU_TANH_NAMES:
            h = self.fc_in(x, activation="gelu_new")
        else:
            h = ACT2FN[self.activation](self.fc_in(x))
        if residual is not None:
            return (self.fc_out(h, residual=residual) if type(self.fc_out) is Linear else self.fc_out(h) + residual)
        return maybe_dropout(self.fc_out(h), self.resid_pdrop, self.training)


class FusedGPTJMLP(GPTJMLP):
    fused = True


class GPTJBlock(nn.Module):
    def __init__(self, config: GPTJConfig) -> None:
        super().__init__()
        inner = config.n_inner if config.n_inner is not None else 4 * config.n_embd
        self.ln_1 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = GPTJAttention(config)
        self.mlp = GPTJMLP(inner, config)

    def _packed_decode_projections(self, x: Tensor):
        """Decode steps (few rows, no grad, fused kernels): q, k, v and fc_in + GeLU read the same LayerNorm output,
        so they run as ONE weight-streaming GEMM over a packed copy of the four weights (rebuilt when any of them
        changes). Returns ``(q, k, v, h)`` or ``None`` when the ordinary per-layer path applies."""
        from ...config import get_config
        from ...ops import cuda_ops
        attn, mlp = self.attn, self.mlp
        layers = (attn.q_proj, attn.k_proj, attn.v_proj, mlp.fc_in)
        if not (attn.fused and mlp.fused and mlp.activation in GELU_TANH_NAMES and get_config().packed_decode):
            return None
        if any(getattr(l, "reversed", False) or not getattr(l, "oslo_fused", False) or getattr(l, "gather_output", False)
               or getattr(l, "sequence_parallel", False) for l in layers):
            return None
        ws = [l.weight for l in layers]
        if any(l.bias is not None for l in layers[:3]) or not cuda_ops.small_m_ok(x, *ws):
            return None
        key = tuple((w.data_ptr(), w._version) for w in ws) + ((mlp.fc_in.bias.data_ptr(), mlp.fc_in.bias._version)
                                                               if mlp.fc_in.bias is not None else ())
        if getattr(self, "_packed_key", None) != key:
            n_qkv = sum(w.size(0) for w in ws[:3])
            self._packed_w = torch.cat([w.detach() for w in ws], dim=0).contiguous()
            fb = mlp.fc_in.bias
            self._packed_b = (torch.cat([fb.new_zeros(n_qkv), fb.detach()]) if fb is not None else None)
            self._packed_key = key
            self._packed_sizes = [w.size(0) for w in ws]
        y = cuda_ops.packed_linear_small_m(x, self._packed_w, self._packed_b, sum(self._packed_sizes[:3]))
        return torch.split(y, self._packed_sizes, dim=-1)

    def _decode_step(self, hidden_states: Tensor, x: Tensor, packed, kw):
        """Whole block for one new token per row on a device-positioned static cache, in six launches: (LayerNorm and
        the packed q/k/v/fc_in GEMV already done) rotary + cache append, decode attention (2), ONE GEMV for
        out_proj and fc_out over [attention | mlp activation] - their sum is what the parallel residual needs -
        ONE all-reduce under tensor parallelism instead of two, and the residual add. Returns ``None`` when the
        general path has to run."""
        from ...ops import cuda_ops
        attn, mlp = self.attn, self.mlp
        cache = kw.get("cache")
        if (cache is None or not getattr(cache, "device_positions", False) or hidden_states.size(1) != 1
                or kw.get("attention_mask") is not None or kw.get("head_mask") is not None
                or kw.get("output_attentions") or self.training or kw.get("layer_id") not in cache.k):
            return None
        rows = hidden_states.size(0)
        out_w, fc_w = attn.out_proj.weight, mlp.fc_out.weight
        if (rows > cuda_ops.SMALL_M_ROWS or attn.out_proj.bias is not None or getattr(attn.out_proj, "reversed", False)
                or getattr(mlp.fc_out, "reversed", False) or out_w.size(0) % 4
                or getattr(attn.out_proj, "sequence_parallel", False)):
            return None
        key = (out_w.data_ptr(), out_w._version, fc_w.data_ptr(), fc_w._version)
        if getattr(self, "_packed2_key", None) != key:
            self._packed2_w = torch.cat([out_w.detach(), fc_w.detach()], dim=1).contiguous()
            self._packed2_key = key
        q, k, v, h = (t.reshape(rows, -1) for t in packed)
        layer = kw["layer_id"]
        kc, vc = cache.k[layer], cache.v[layer]
        rd = attn.rotary_dim if attn.rotary_dim is not None else attn.head_dim
        q_rot = cuda_ops.rotary_append(q, k, v, kc, vc, cache.lengths_dev, cache.write_index, rd)
        o = ops.decode_attention(q_rot, kc, vc, cache.lengths_next, attn.scale, attn.window)
        mpu = getattr(attn.out_proj, "mpu", None)
        tp = mpu.tp if mpu is not None else 1
        fc_bias = mlp.fc_out.bias
        if rows <= cuda_ops.GEMV_ROWS:
            # bias and residual enter the sum exactly once: on tensor-parallel rank 0, before the all-reduce
            first = tp == 1 or mpu.tp_rank == 0
            z = cuda_ops.gemv_two_inputs(o.reshape(rows, -1), h, self._packed2_w, fc_bias if first else None,
                                         hidden_states.reshape(rows, -1) if first else None)
            if tp > 1:
                z = mpu._reduce(z)
            return z.view_as(hidden_states), None, None
        # more rows than the CUDA cores can feed from HBM: tensor-core split-k GEMM over the joined input
        z = cuda_ops.packed_linear_small_m(torch.cat([o.reshape(rows, -1), h], dim=1), self._packed2_w, None, -1)
        if tp > 1:
            z = mpu._reduce(z)
        z = z.view_as(hidden_states)
        if fc_bias is not None:
            z = z + fc_bias
        return z + hidden_states, None, None

    def _tp_shared_input(self, x: Tensor):
        """``(q, k, v, h)`` through ``fused_tp.tp_block_input`` when the four layers are plain column-parallel shards
        (``[out_shard, in]`` weights, no gathered output, no sequence parallelism, bias only on fc_in) in training."""
        from ...parallel.layers import ColumnParallelLinear
        attn, mlp = self.attn, self.mlp
        layers = (attn.q_proj, attn.k_proj, attn.v_proj, mlp.fc_in)
        if not (get_config().tp_shared_input_grad and torch.is_grad_enabled() and mlp.activation in GELU_TANH_NAMES
                and attn.fused == mlp.fused):
            return None
        for l in layers:
            if not (type(l) is ColumnParallelLinear and not l.reversed and not l.gather_output and not l.sequence_parallel
                    and l.mpu is not None and l.mpu.tp > 1 and l.oslo_fused == attn.fused):
                return None
        if any(l.bias is not None for l in layers[:3]):
            return None
        if x.is_cuda:
            from ...ops import cuda_ops
            if not (attn.fused and cuda_ops.qkv_linear_ok(x, *(l.weight for l in layers))):
                return None
        elif attn.fused:
            return None
        from ...parallel.fused_tp import tp_block_input
        return tp_block_input(x, attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight, mlp.fc_in.weight,
                              mlp.fc_in.bias, attn.q_proj.mpu)

    def forward(self, hidden_states: Tensor, **kw):
        x = self.ln_1(hidden_states)
        packed = self._packed_decode_projections(x) if x.is_cuda else None
        if packed is not None:
            fast = self._decode_step(hidden_states, x, packed, kw)
            if fast is not None:
                return fast
            a, present, probs = self.attn(x, qkv=packed[:3], **kw)
            m = self.mlp(x, h=packed[3])
            return a + m + hidden_states, present, probs
        no_dropout = not self.training or (self.attn.resid_pdrop == 0.0 and self.mlp.resid_pdrop == 0.0)
        if (no_dropout and x.is_cuda and self.attn.fused and type(self.attn.out_proj) is Linear
                and kw.get("seq_shape") is None and get_config().block_fusion):
            # hidden + attn + mlp with both additions inside GEMM epilogues: out_proj adds the block input, fc_out adds
            # that sum
            a, present, probs = self.attn(x, residual=hidden_states, **kw)
            return self.mlp(x, residual=a), present, probs
        sp = kw.get("seq_shape") is not None
        if (no_dropout and get_config().block_fusion
                and isinstance(self.attn.out_proj, RowParallelLinear) and isinstance(self.mlp.fc_out, RowParallelLinear)
                and self.attn.out_proj.bias is None and getattr(self.attn.out_proj, "mpu", None) is not None
                and self.attn.out_proj.mpu.tp > 1 and self.attn.out_proj.sequence_parallel == sp
                and self.mlp.fc_out.sequence_parallel == sp
                and (not sp or not x.is_cuda or get_config().tp_shared_reduction_sp)):
            # tensor parallel: attention projection and fc_out are both row-parallel and their sum is all the block
            # needs, so ONE collective reduces both (the projection's partial sum rides along in fc_out's kernel)
            pre = None if sp else self._tp_shared_input(x)
            if pre is not None:   # q / k / v / fc_in as one node: ONE all-reduce of the block's input gradient too
                a_part, present, probs = self.attn(x, qkv=pre[:3], partial_only=True, **kw)
                return self.mlp(x, h=pre[3], partial=a_part, residual=None if sp else hidden_states), present, probs
            a_part, present, probs = self.attn(x, partial_only=True, **kw)
            if sp:
                return self.mlp(x, partial=a_part) + hidden_states, present, probs
            return self.mlp(x, partial=a_part, residual=hidden_states), present, probs
        a, present, probs = self.attn(x, **kw)
        m = self.mlp(x)
        return a + m + hidden_states, present, probs


class GPTJPreTrainedModel(PreTrainedModel):
    config_class = GPTJConfig
    base_model_prefix = "transformer"

    def get_layer_policies(self):
        return [GPTJLayerPolicy]


class GPTJModel(DecoderBackbone, GPTJPreTrainedModel):
    def __init__(self, config: GPTJConfig) -> None:
        super().__init__(config)
        self.embed_dim = config.n_embd
        self.wte = Embedding(config.vocab_size, self.embed_dim)
        self.embd_pdrop = config.embd_pdrop
        self.h = nn.ModuleList([GPTJBlock(config) for _ in range(config.n_layer)])
        self.ln_f = LayerNorm(self.embed_dim, eps=config.layer_norm_epsilon)
        self.post_init()

    def embed(self, input_ids, position_ids, token_type_ids, inputs_embeds):
        hs = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        if token_type_ids is not None:
            hs = hs + self.wte(token_type_ids)
        return maybe_dropout(hs, self.embd_pdrop, self.training)


class GPTJForCausalLM(CausalLMHeadMixin, GPTJPreTrainedModel):
    _keys_to_ignore_on_load_missing = [r"attn.masked_bias", r"attn.bias"]

    def __init__(self, config: GPTJConfig) -> None:
        super().__init__(config)
        self.transformer = GPTJModel(config)
        self.lm_head = Linear(config.n_embd, config.vocab_size)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        # vocabulary-sharded head (the reference keeps it whole on every rank,
        # oslo/models/gptj/modeling_gptj.py:734-742); split checkpoints still store it whole.
        return [Layer(module=self.lm_head, weight=self.lm_head.weight, bias=self.lm_head.bias,
                      replace={Linear: "vocab_head"}, parallel=True, gather_output=True)]


class GPTJForSequenceClassification(SequenceClassificationMixin, GPTJPreTrainedModel):
    def __init__(self, config: GPTJConfig) -> None:
        super().__init__(config)
        self.num_labels = config.num_labels
        self.transformer = GPTJModel(config)
        self.score = Linear(config.n_embd, self.num_labels, bias=False)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        return [Layer(module=self.score, weight=self.score.weight, parallel=False)]


class GPTJLayerPolicy(LayerPolicy):
    @staticmethod
    def reduce_arguments(layer, world_size, config):
        layer.attn.embed_dim = config.n_embd // world_size
        layer.attn.num_attention_heads = config.n_head // world_size

    @staticmethod
    def fused_modules():
        return {GPTJAttention: FusedGPTJAttention, GPTJMLP: FusedGPTJMLP}

    @staticmethod
    def attn_qkv(layer, config):
        return [Layer(module=m, weight=m.weight, bias=None, replace={Linear: "column"})
                for m in (layer.attn.q_proj, layer.attn.k_proj, layer.attn.v_proj)]

    @staticmethod
    def attn_out(layer, config):
        m = layer.attn.out_proj
        return [Layer(module=m, weight=m.weight, bias=None, replace={Linear: "row"})]

    @staticmethod
    def attn_norm(layer, config):
        return [Layer(module=layer.ln_1, weight=layer.ln_1.weight, bias=layer.ln_1.bias, parallel=False)]

    @staticmethod
    def mlp_in(layer, config):
        m = layer.mlp.fc_in
        return [Layer(module=m, weight=m.weight, bias=m.bias, replace={Linear: "column"})]

    @staticmethod
    def mlp_out(layer, config):
        m = layer.mlp.fc_out
        return [Layer(module=m, weight=m.weight, bias=m.bias, replace={Linear: "row"})]

    @staticmethod
    def word_embedding(model, config):
        wte = model.base_model.wte
        return [Layer(module=wte, weight=wte.weight, replace={Embedding: "vocab_embedding"})]

    @staticmethod
    def block_layers(model, config):
        return list(model.base_model.h)

    @staticmethod
    def postblock_layers(model, config):
        ln = model.base_model.ln_f
        return [Layer(module=ln, weight=ln.weight, bias=ln.bias, parallel=False)]

    @staticmethod
    def original_layer_class():
        return GPTJBlock
