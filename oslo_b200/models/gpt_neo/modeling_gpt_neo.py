"""GPT-Neo: alternating global / local (sliding window) attention, unscaled scores, tied LM head.

The local layers keep keys ``q_pos - window < k_pos <= q_pos`` (the reference builds this as a
mask buffer ``bias ^ tril(bias, -window)``, oslo/models/gpt_neo/modeling_gpt_neo.py:150-160); here
the window is an argument of the attention kernels, so local layers only visit the blocks inside
the window and, unlike the reference (``GPTNeoLocalSelfAttention`` is skipped by ``fuse()``,
:270-272), they are fused too.
"""
from __future__ import annotations

from typing import List

import torch.nn as nn
from torch import Tensor

from ...fused_kernels_utils import ACT2FN, GELU_TANH_NAMES
from ...modeling_utils import PretrainedConfig, PreTrainedModel
from ...parallel.layers import Embedding, LayerNorm, Linear
from ...parallel.mpu import Layer, LayerPolicy
from ..common import (AttentionCore, CausalLMHeadMixin, DecoderBackbone, SequenceClassificationMixin,
                      maybe_dropout, merge_heads, split_heads, to_batch_seq, to_token_rows)


class GPTNeoConfig(PretrainedConfig):
    model_type = "gpt_neo"
    attribute_map = {"num_attention_heads": "num_heads", "num_hidden_layers": "num_layers",
                     "n_embd": "hidden_size", "n_layer": "num_layers", "n_head": "num_heads",
                     "n_positions": "max_position_embeddings"}

    def __init__(self, vocab_size=50257, max_position_embeddings=2048, hidden_size=2048, num_layers=24,
                 attention_types=None, num_heads=16, intermediate_size=None, window_size=256,
                 activation_function="gelu_new", resid_dropout=0.0, embed_dropout=0.0, attention_dropout=0.0,
                 layer_norm_epsilon=1e-5, initializer_range=0.02, summary_type="cls_index", summary_use_proj=True,
                 summary_activation=None, summary_proj_to_labels=True, summary_first_dropout=0.1, use_cache=True,
                 bos_token_id=50256, eos_token_id=50256, **kwargs):
        if attention_types is None:
            attention_types = [[["global", "local"], num_layers // 2]] if num_layers % 2 == 0 else [[["global"], num_layers]]
        self.vocab_size, self.max_position_embeddings, self.hidden_size = vocab_size, max_position_embeddings, hidden_size
        self.num_layers, self.num_heads, self.intermediate_size, self.window_size = num_layers, num_heads, intermediate_size, window_size
        self.activation_function = activation_function
        self.resid_dropout, self.embed_dropout, self.attention_dropout = resid_dropout, embed_dropout, attention_dropout
        self.layer_norm_epsilon, self.initializer_range = layer_norm_epsilon, initializer_range
        self.summary_type, self.summary_use_proj, self.summary_activation = summary_type, summary_use_proj, summary_activation
        self.summary_proj_to_labels, self.summary_first_dropout = summary_proj_to_labels, summary_first_dropout
        self.attention_types = attention_types
        self.attention_layers = self.expand_attention_types_params(attention_types)
        if len(self.attention_layers) != num_layers:
            raise ValueError(
                f"attention_types expands to {len(self.attention_layers)} layers but num_layers is {num_layers}")
        kwargs.pop("attention_layers", None)
        super().__init__(use_cache=use_cache, bos_token_id=bos_token_id, eos_token_id=eos_token_id, **kwargs)

    @staticmethod
    def expand_attention_types_params(attention_types) -> List[str]:
        out: List[str] = []
        for kinds, repeat in attention_types:
            for _ in range(repeat):
                out.extend(kinds)
        return out


class GPTNeoSelfAttention(AttentionCore):
    def __init__(self, config: GPTNeoConfig, attention_type: str = "global") -> None:
        super().__init__()
        self.embed_dim = config.hidden_size
        self.num_heads = config.num_heads
        self.head_dim = self.embed_dim // self.num_heads
        if self.head_dim * self.num_heads != self.embed_dim:
            raise ValueError("hidden_size must be divisible by num_heads")
        self.scale = 1.0  # GPT-Neo does not scale scores
        self.window = config.window_size if attention_type == "local" else None
        self.attn_pdrop, self.resid_pdrop = float(config.attention_dropout), float(config.resid_dropout)
        self.k_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.v_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.q_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.out_proj = Linear(self.embed_dim, self.embed_dim, bias=True)

    def forward(self, hidden_states: Tensor, layer_past=None, attention_mask=None, position_ids=None,
                head_mask=None, use_cache=False, output_attentions=False, cache=None, layer_id=0, seq_shape=None):
        nh, hd = self.num_heads, self.head_dim
        q = split_heads(to_batch_seq(self.q_proj(hidden_states), seq_shape), nh, hd)
        k = split_heads(to_batch_seq(self.k_proj(hidden_states), seq_shape), nh, hd)
        v = split_heads(to_batch_seq(self.v_proj(hidden_states), seq_shape), nh, hd)
        out, present, probs = self.attend_with_cache(q, k, v, layer_past, cache, layer_id, attention_mask,
                                                     use_cache, output_attentions, head_mask)
        out = self.out_proj(to_token_rows(merge_heads(out), seq_shape))
        return maybe_dropout(out, self.resid_pdrop, self.training), present, probs


class GPTNeoLocalSelfAttention(GPTNeoSelfAttention):
    """Sliding-window layers; a separate class so ``fuse([GPTNeoSelfAttention])`` can leave them out."""

    def __init__(self, config: GPTNeoConfig) -> None:
        super().__init__(config, "local")


class FusedGPTNeoSelfAttention(GPTNeoSelfAttention):
    fused = True


class FusedGPTNeoLocalSelfAttention(GPTNeoLocalSelfAttention):
    fused = True


class GPTNeoAttention(nn.Module):
    def __init__(self, config: GPTNeoConfig, layer_id: int = 0) -> None:
        super().__init__()
        self.attention_type = config.attention_layers[layer_id]
        if self.attention_type == "global":
            self.attention = GPTNeoSelfAttention(config)
        elif self.attention_type == "local":
            self.attention = GPTNeoLocalSelfAttention(config)
        else:
            raise NotImplementedError(f"unknown attention type {self.attention_type!r}")

    def forward(self, hidden_states, **kw):
        return self.attention(hidden_states, **kw)


class GPTNeoMLP(nn.Module):
    fused = False

    def __init__(self, intermediate_size: int, config: GPTNeoConfig) -> None:
        super().__init__()
        self.c_fc = Linear(config.hidden_size, intermediate_size)
        self.c_proj = Linear(intermediate_size, config.hidden_size)
        self.activation = config.activation_function
        self.resid_pdrop = float(config.resid_dropout)

    def forward(self, x: Tensor) -> Tensor:
        if self.fused and self.activation in GELU_TANH_NAMES:
            h = self.c_fc(x, activation="gelu_new")
        else:
            h = ACT2FN[self.activation](self.c_fc(x))
        return maybe_dropout(self.c_proj(h), self.resid_pdrop, self.training)


class FusedGPTNeoMLP(GPTNeoMLP):
    fused = True


class GPTNeoBlock(nn.Module):
    def __init__(self, config: GPTNeoConfig, layer_id: int) -> None:
        super().__init__()
        inner = config.intermediate_size if config.intermediate_size is not None else 4 * config.hidden_size
        self.ln_1 = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.attn = GPTNeoAttention(config, layer_id)
        self.ln_2 = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp = GPTNeoMLP(inner, config)

    def forward(self, hidden_states: Tensor, **kw):
        a, present, probs = self.attn(self.ln_1(hidden_states), **kw)
        hidden_states = a + hidden_states
        hidden_states = hidden_states + self.mlp(self.ln_2(hidden_states))
        return hidden_states, present, probs


class GPTNeoPreTrainedModel(PreTrainedModel):
    config_class = GPTNeoConfig
    base_model_prefix = "transformer"

    def get_layer_policies(self):
        return [GPTNeoLayerPolicy]


class GPTNeoModel(DecoderBackbone, GPTNeoPreTrainedModel):
    def __init__(self, config: GPTNeoConfig) -> None:
        super().__init__(config)
        self.embed_dim = config.hidden_size
        self.wte = Embedding(config.vocab_size, self.embed_dim)
        self.wpe = Embedding(config.max_position_embeddings, self.embed_dim)
        self.embd_pdrop = float(config.embed_dropout)
        self.h = nn.ModuleList([GPTNeoBlock(config, layer_id=i) for i in range(config.num_layers)])
        self.ln_f = LayerNorm(self.embed_dim, eps=config.layer_norm_epsilon)
        self.post_init()

    def embed(self, input_ids, position_ids, token_type_ids, inputs_embeds):
        hs = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        hs = hs + self.wpe(position_ids)
        if token_type_ids is not None:
            hs = hs + self.wte(token_type_ids)
        return maybe_dropout(hs, self.embd_pdrop, self.training)


class GPTNeoForCausalLM(CausalLMHeadMixin, GPTNeoPreTrainedModel):
    _keys_to_ignore_on_load_missing = [r"h\.\d+\.attn\.masked_bias", r"lm_head.weight", r"h\.\d+\.attn\.attention\.bias"]
    _keys_to_ignore_on_save = ["lm_head.weight"]

    def __init__(self, config: GPTNeoConfig) -> None:
        super().__init__(config)
        self.transformer = GPTNeoModel(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        wte = self.transformer.wte
        return [Layer(module=self.lm_head, weight=self.lm_head.weight, replace={Linear: "vocab_head"},
                      parallel=False, gather_output=True, tied_embedding=wte)]


class GPTNeoForSequenceClassification(SequenceClassificationMixin, GPTNeoPreTrainedModel):
    _keys_to_ignore_on_load_missing = [r"h\.\d+\.attn\.masked_bias", r"lm_head.weight"]

    def __init__(self, config: GPTNeoConfig) -> None:
        super().__init__(config)
        self.num_labels = config.num_labels
        self.transformer = GPTNeoModel(config)
        self.score = Linear(config.hidden_size, self.num_labels, bias=False)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        return [Layer(module=self.score, weight=self.score.weight, parallel=False)]


class GPTNeoLayerPolicy(LayerPolicy):
    @staticmethod
    def reduce_arguments(layer, world_size, config):
        a = layer.attn.attention
        a.embed_dim = config.hidden_size // world_size
        a.num_heads = config.num_heads // world_size

    @staticmethod
    def fused_modules():
        return {GPTNeoSelfAttention: FusedGPTNeoSelfAttention,
                GPTNeoLocalSelfAttention: FusedGPTNeoLocalSelfAttention, GPTNeoMLP: FusedGPTNeoMLP}

    @staticmethod
    def attn_qkv(layer, config):
        a = layer.attn.attention
        return [Layer(module=m, weight=m.weight, bias=None, replace={Linear: "column"})
                for m in (a.q_proj, a.k_proj, a.v_proj)]

    @staticmethod
    def attn_out(layer, config):
        m = layer.attn.attention.out_proj
        return [Layer(module=m, weight=m.weight, bias=m.bias, replace={Linear: "row"})]

    @staticmethod
    def attn_norm(layer, config):
        return [Layer(module=layer.ln_1, weight=layer.ln_1.weight, bias=layer.ln_1.bias, parallel=False)]

    @staticmethod
    def mlp_in(layer, config):
        m = layer.mlp.c_fc
        return [Layer(module=m, weight=m.weight, bias=m.bias, replace={Linear: "column"})]

    @staticmethod
    def mlp_out(layer, config):
        m = layer.mlp.c_proj
        return [Layer(module=m, weight=m.weight, bias=m.bias, replace={Linear: "row"})]

    @staticmethod
    def mlp_norm(layer, config):
        return [Layer(module=layer.ln_2, weight=layer.ln_2.weight, bias=layer.ln_2.bias, parallel=False)]

    @staticmethod
    def word_embedding(model, config):
        wte = model.base_model.wte
        return [Layer(module=wte, weight=wte.weight, replace={Embedding: "vocab_embedding"})]

    @staticmethod
    def preblock_layers(model, config):
        wpe = model.base_model.wpe
        return [Layer(module=wpe, weight=wpe.weight, parallel=False)]

    @staticmethod
    def block_layers(model, config):
        return list(model.base_model.h)

    @staticmethod
    def postblock_layers(model, config):
        ln = model.base_model.ln_f
        return [Layer(module=ln, weight=ln.weight, bias=ln.bias, parallel=False)]

    @staticmethod
    def original_layer_class():
        return GPTNeoBlock
