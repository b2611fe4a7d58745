"""GPT-2: learned position embeddings, fused ``c_attn`` Conv1D projection, tied LM head.

Covers the reference's GPT-2 zoo (oslo/models/gpt2/modeling_gpt2.py): base model, LM head,
double heads, sequence and token classification, optional cross-attention,
``scale_attn_by_inverse_layer_idx`` and head pruning. Attention is computed with fp32 scores,
which also makes the ``reorder_and_upcast_attn`` flag a no-op.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ... import ops
from ...fused_kernels_utils import ACT2FN, GELU_TANH_NAMES, FusedScaleMaskSoftmax
from ...modeling_utils import (GPT2DoubleHeadsModelOutput, PretrainedConfig, PreTrainedModel,
                               TokenClassifierOutput)
from ...parallel.layers import Conv1D, Embedding, LayerNorm, Linear
from ...parallel.mpu import Layer, LayerPolicy
from ..common import (AttentionCore, CausalLMHeadMixin, DecoderBackbone, SequenceClassificationMixin,
                      maybe_dropout, merge_heads, split_heads, to_batch_seq, to_token_rows)


class GPT2Config(PretrainedConfig):
    model_type = "gpt2"
    attribute_map = {"hidden_size": "n_embd", "max_position_embeddings": "n_positions",
                     "num_attention_heads": "n_head", "num_hidden_layers": "n_layer"}

    def __init__(self, vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=None,
                 activation_function="gelu_new", resid_pdrop=0.1, embd_pdrop=0.1, attn_pdrop=0.1,
                 layer_norm_epsilon=1e-5, initializer_range=0.02, summary_type="cls_index", summary_use_proj=True,
                 summary_activation=None, summary_proj_to_labels=True, summary_first_dropout=0.1,
                 scale_attn_weights=True, use_cache=True, bos_token_id=50256, eos_token_id=50256,
                 scale_attn_by_inverse_layer_idx=False, reorder_and_upcast_attn=False,
                 add_cross_attention=False, **kwargs):
        self.vocab_size, self.n_positions, self.n_embd, self.n_layer, self.n_head = vocab_size, n_positions, n_embd, n_layer, n_head
        self.n_inner, self.activation_function = n_inner, activation_function
        self.resid_pdrop, self.embd_pdrop, self.attn_pdrop = resid_pdrop, embd_pdrop, attn_pdrop
        self.layer_norm_epsilon, self.initializer_range = layer_norm_epsilon, initializer_range
        self.summary_type, self.summary_use_proj, self.summary_activation = summary_type, summary_use_proj, summary_activation
        self.summary_proj_to_labels, self.summary_first_dropout = summary_proj_to_labels, summary_first_dropout
        self.scale_attn_weights = scale_attn_weights
        self.scale_attn_by_inverse_layer_idx = scale_attn_by_inverse_layer_idx
        self.reorder_and_upcast_attn = reorder_and_upcast_attn
        self.add_cross_attention = add_cross_attention
        super().__init__(use_cache=use_cache, bos_token_id=bos_token_id, eos_token_id=eos_token_id, **kwargs)


class GPT2Attention(AttentionCore):
    def __init__(self, config: GPT2Config, is_cross_attention: bool = False, layer_idx: Optional[int] = None) -> None:
        super().__init__()
        self.embed_dim = config.n_embd
        self.num_heads = config.n_head
        self.head_dim = self.embed_dim // self.num_heads
        self.split_size = self.embed_dim
        if self.head_dim * self.num_heads != self.embed_dim:
            raise ValueError("n_embd must be divisible by n_head")
        self.is_cross_attention = is_cross_attention
        self.layer_idx = layer_idx
        scale = 1.0 / math.sqrt(self.head_dim) if config.scale_attn_weights else 1.0
        if config.scale_attn_by_inverse_layer_idx and layer_idx is not None:
            scale /= float(layer_idx + 1)
        self.scale = scale
        if is_cross_attention:
            self.c_attn = Conv1D(2 * self.embed_dim, self.embed_dim)
            self.q_attn = Conv1D(self.embed_dim, self.embed_dim)
        else:
            self.c_attn = Conv1D(3 * self.embed_dim, self.embed_dim)
        self.c_proj = Conv1D(self.embed_dim, self.embed_dim)
        self.attn_pdrop, self.resid_pdrop = config.attn_pdrop, config.resid_pdrop
        self.pruned_heads = set()

    def prune_heads(self, heads) -> None:
        heads = set(heads) - self.pruned_heads
        if not heads:
            return
        keep_heads = [h for h in range(self.num_heads) if h not in heads]
        idx = torch.cat([torch.arange(h * self.head_dim, (h + 1) * self.head_dim) for h in keep_heads])
        idx_attn = torch.cat([idx, idx + self.split_size, idx + 2 * self.split_size])
        self.c_attn.weight = nn.Parameter(self.c_attn.weight.data.index_select(1, idx_attn).clone())
        self.c_attn.bias = nn.Parameter(self.c_attn.bias.data.index_select(0, idx_attn).clone())
        self.c_proj.weight = nn.Parameter(self.c_proj.weight.data.index_select(0, idx).clone())
        self.split_size = (self.split_size // self.num_heads) * (self.num_heads - len(heads))
        self.num_heads -= len(heads)
        self.pruned_heads |= heads

    def forward(self, hidden_states: Tensor, layer_past=None, attention_mask=None, position_ids=None,
                head_mask=None, use_cache=False, output_attentions=False, cache=None, layer_id=0,
                encoder_hidden_states=None, encoder_attention_mask=None, seq_shape=None):
        nh, hd = self.num_heads, self.head_dim
        if encoder_hidden_states is not None:
            if not self.is_cross_attention:
                raise ValueError("cross-attention needs GPT2Attention(is_cross_attention=True)")
            q = split_heads(self.q_attn(hidden_states), nh, hd)
            k, v = self.c_attn(encoder_hidden_states).split(self.split_size, dim=2)
            k, v = split_heads(k, nh, hd), split_heads(v, nh, hd)
            out, probs = self._cross_attention(q, k, v, encoder_attention_mask, head_mask)
            present = None
        else:
            q, k, v = to_batch_seq(self.c_attn(hidden_states), seq_shape).split(self.split_size, dim=2)
            q, k, v = split_heads(q, nh, hd), split_heads(k, nh, hd), split_heads(v, nh, hd)
            out, present, probs = self.attend_with_cache(q, k, v, layer_past, cache, layer_id, attention_mask,
                                                         use_cache, output_attentions, head_mask)
        out = self.c_proj(to_token_rows(merge_heads(out), seq_shape))
        return maybe_dropout(out, self.resid_pdrop, self.training), present, probs

    def _cross_attention(self, q, k, v, encoder_attention_mask, head_mask):
        """Non-causal attention over encoder states; padded keys get -10000 before the softmax."""
        scores = torch.matmul(q, k.transpose(-1, -2))
        b, _, sq, sk = scores.shape
        if encoder_attention_mask is None:
            mask = torch.zeros(b, 1, sq, sk, dtype=torch.uint8, device=q.device)
        else:
            mask = (encoder_attention_mask.view(b, 1, 1, sk) == 0).expand(b, 1, sq, sk).to(torch.uint8)
        if self.fused:
            probs = FusedScaleMaskSoftmax.apply(scores, mask, self.scale, False)
        else:
            probs = ops.reference.scaled_masked_softmax(scores, mask, self.scale)
        probs = maybe_dropout(probs, self.attn_pdrop, self.training)
        if head_mask is not None:
            probs = probs * head_mask
        return torch.matmul(probs, v), probs


class FusedGPT2Attention(GPT2Attention):
    fused = True


class GPT2MLP(nn.Module):
    fused = False

    def __init__(self, intermediate_size: int, config: GPT2Config) -> None:
        super().__init__()
        self.c_fc = Conv1D(intermediate_size, config.n_embd)
        self.c_proj = Conv1D(config.n_embd, intermediate_size)
        self.activation = config.activation_function
        self.resid_pdrop = config.resid_pdrop

    def forward(self, x: Tensor) -> Tensor:
        if self.fused and self.activation in GELU_TANH_NAMES:
            h = self.c_fc(x, activation="gelu_new")
        else:
            h = ACT2FN[self.activation](self.c_fc(x))
        return maybe_dropout(self.c_proj(h), self.resid_pdrop, self.training)


class FusedGPT2MLP(GPT2MLP):
    fused = True


class GPT2Block(nn.Module):
    def __init__(self, config: GPT2Config, layer_idx: Optional[int] = None) -> None:
        super().__init__()
        inner = config.n_inner if config.n_inner is not None else 4 * config.n_embd
        self.ln_1 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = GPT2Attention(config, layer_idx=layer_idx)
        self.ln_2 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        if config.add_cross_attention:
            self.crossattention = GPT2Attention(config, is_cross_attention=True, layer_idx=layer_idx)
            self.ln_cross_attn = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.mlp = GPT2MLP(inner, config)

    def forward(self, hidden_states: Tensor, encoder_hidden_states=None, encoder_attention_mask=None, **kw):
        a, present, probs = self.attn(self.ln_1(hidden_states), **kw)
        hidden_states = a + hidden_states
        if encoder_hidden_states is not None:
            if not hasattr(self, "crossattention"):
                raise ValueError("encoder_hidden_states given but config.add_cross_attention is False")
            c, _, _ = self.crossattention(self.ln_cross_attn(hidden_states), head_mask=kw.get("head_mask"),
                                          encoder_hidden_states=encoder_hidden_states,
                                          encoder_attention_mask=encoder_attention_mask)
            hidden_states = hidden_states + c
        hidden_states = hidden_states + self.mlp(self.ln_2(hidden_states))
        return hidden_states, present, probs


class GPT2PreTrainedModel(PreTrainedModel):
    config_class = GPT2Config
    base_model_prefix = "transformer"

    def _init_weights(self, module: nn.Module) -> None:
        super()._init_weights(module)
        if isinstance(module, (GPT2Attention, GPT2MLP)):
            std = self.config.initializer_range / math.sqrt(2 * self.config.n_layer)
            module.c_proj.weight.data.normal_(mean=0.0, std=std)

    def get_layer_policies(self):
        return [GPT2LayerPolicy]


class GPT2Model(DecoderBackbone, GPT2PreTrainedModel):
    def __init__(self, config: GPT2Config) -> None:
        super().__init__(config)
        self.embed_dim = config.n_embd
        self.wte = Embedding(config.vocab_size, self.embed_dim)
        self.wpe = Embedding(config.n_positions, self.embed_dim)
        self.embd_pdrop = config.embd_pdrop
        self.h = nn.ModuleList([GPT2Block(config, layer_idx=i) for i in range(config.n_layer)])
        self.ln_f = LayerNorm(self.embed_dim, eps=config.layer_norm_epsilon)
        self.post_init()

    def embed(self, input_ids, position_ids, token_type_ids, inputs_embeds):
        hs = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        hs = hs + self.wpe(position_ids)
        if token_type_ids is not None:
            hs = hs + self.wte(token_type_ids)
        return maybe_dropout(hs, self.embd_pdrop, self.training)

    def _prune_heads(self, heads_to_prune) -> None:
        for layer, heads in heads_to_prune.items():
            self.h[layer].attn.prune_heads(heads)

    prune_heads = _prune_heads


def _tied_head_layer(model) -> Layer:
    wte = model.transformer.wte
    return Layer(module=model.lm_head, weight=model.lm_head.weight, replace={Linear: "vocab_head"},
                 parallel=False, gather_output=True, tied_embedding=wte)


class GPT2LMHeadModel(CausalLMHeadMixin, GPT2PreTrainedModel):
    _keys_to_ignore_on_load_missing = [r"attn.masked_bias", r"attn.bias", r"lm_head.weight"]

    def __init__(self, config: GPT2Config) -> None:
        super().__init__(config)
        self.transformer = GPT2Model(config)
        self.lm_head = Linear(config.n_embd, config.vocab_size, bias=False)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        return [_tied_head_layer(self)]


class SequenceSummary(nn.Module):
    """Pools one hidden state per sequence (``summary_type``: last / first / mean / cls_index) and projects it."""

    def __init__(self, config: GPT2Config) -> None:
        super().__init__()
        self.summary_type = getattr(config, "summary_type", "last")
        self.summary = nn.Identity()
        if getattr(config, "summary_use_proj", False):
            n = config.num_labels if (getattr(config, "summary_proj_to_labels", False) and config.num_labels > 0) else config.hidden_size
            self.summary = Linear(config.hidden_size, n)
        act = getattr(config, "summary_activation", None)
        self.activation = ACT2FN[act] if act else nn.Identity()
        self.first_dropout = nn.Dropout(getattr(config, "summary_first_dropout", 0.0) or 0.0)

    def forward(self, hidden_states: Tensor, cls_index: Optional[Tensor] = None) -> Tensor:
        if self.summary_type == "last":
            out = hidden_states[:, -1]
        elif self.summary_type == "first":
            out = hidden_states[:, 0]
        elif self.summary_type == "mean":
            out = hidden_states.mean(dim=1)
        elif self.summary_type == "cls_index":
            if cls_index is None:
                cls_index = torch.full_like(hidden_states[..., :1, :], hidden_states.shape[-2] - 1, dtype=torch.long)
            else:
                cls_index = cls_index.unsqueeze(-1).unsqueeze(-1)
                cls_index = cls_index.expand((-1,) * (cls_index.dim() - 1) + (hidden_states.size(-1),))
            out = hidden_states.gather(-2, cls_index).squeeze(-2)
        else:
            raise NotImplementedError(self.summary_type)
        return self.activation(self.summary(self.first_dropout(out)))


class GPT2DoubleHeadsModel(CausalLMHeadMixin, GPT2PreTrainedModel):
    """LM head + multiple-choice head; inputs are ``[batch, choices, seq]``."""

    _keys_to_ignore_on_load_missing = [r"attn.masked_bias", r"attn.bias", r"lm_head.weight"]

    def __init__(self, config: GPT2Config) -> None:
        super().__init__(config)
        config.num_labels = 1
        self.transformer = GPT2Model(config)
        self.lm_head = Linear(config.n_embd, config.vocab_size, bias=False)
        self.multiple_choice_head = SequenceSummary(config)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        s = self.multiple_choice_head.summary
        extra = [Layer(module=s, weight=s.weight, bias=s.bias, parallel=False)] if isinstance(s, Linear) else []
        return [_tied_head_layer(self)] + extra

    def preblock_fn(self, input_ids=None, mc_token_ids=None, mc_labels=None, **kw):
        kw["_in_shape"] = tuple(input_ids.shape) if input_ids is not None else None
        kw["mc_token_ids"], kw["mc_labels"] = mc_token_ids, mc_labels
        return self.transformer.preblock_fn(input_ids=input_ids, **kw)

    def prepare_fn(self, input_ids=None, mc_token_ids=None, mc_labels=None, **kw):
        """What ``preblock_fn`` records about the inputs, for pipeline stages that do not own the embeddings."""
        kw["_in_shape"] = tuple(input_ids.shape) if input_ids is not None else None
        kw["mc_token_ids"], kw["mc_labels"] = mc_token_ids, mc_labels
        return self.transformer.prepare_fn(input_ids=input_ids, **kw)

    def head_fn(self, **kw):
        labels = kw.pop("labels", None)
        kw = CausalLMHeadMixin.head_fn(self, **kw)
        kw["labels"] = labels
        shape = kw.get("_in_shape")
        hs = kw["hidden_states"]
        if shape is not None and len(shape) == 3:
            hs = hs.view(shape[0], shape[1], shape[2], -1)
            kw["logits"] = kw["logits"].view(shape[0], shape[1], shape[2], -1)
        kw["mc_logits"] = self.multiple_choice_head(hs, kw.get("mc_token_ids")).squeeze(-1)
        return kw

    def loss_fn(self, **kw):
        kw["mc_loss"] = None
        if kw.get("mc_labels") is not None:
            mc = kw["mc_logits"]
            kw["mc_loss"] = F.cross_entropy(mc.view(-1, mc.size(-1)).float(), kw["mc_labels"].view(-1))
        kw["loss"] = None
        if kw.get("labels") is not None:
            lg = kw["logits"]
            shift = lg[..., :-1, :].contiguous()
            tgt = kw["labels"][..., 1:].contiguous()
            kw["loss"] = F.cross_entropy(shift.view(-1, shift.size(-1)).float(), tgt.view(-1))
        return kw

    def organize_fn(self, **kw):
        out = GPT2DoubleHeadsModelOutput(
            loss=kw.get("loss"), mc_loss=kw.get("mc_loss"), logits=kw.get("logits"), mc_logits=kw.get("mc_logits"),
            past_key_values=self.transformer.collect_past(kw),
            hidden_states=tuple(kw["all_hidden_states"]) if kw["all_hidden_states"] is not None else None,
            attentions=tuple(kw["all_attentions"]) if kw["all_attentions"] is not None else None)
        return out if kw["return_dict"] else out.to_tuple()


class GPT2ForSequenceClassification(SequenceClassificationMixin, GPT2PreTrainedModel):
    _keys_to_ignore_on_load_missing = [r"h\.\d+\.attn\.masked_bias", r"lm_head\.weight"]

    def __init__(self, config: GPT2Config) -> None:
        super().__init__(config)
        self.num_labels = config.num_labels
        self.transformer = GPT2Model(config)
        self.score = Linear(config.n_embd, self.num_labels, bias=False)
        self.post_init()

    def get_head_layers(self) -> List[Layer]:
        return [Layer(module=self.score, weight=self.score.weight, parallel=False)]


class GPT2ForTokenClassification(GPT2PreTrainedModel):
    def __init__(self, config: GPT2Config) -> None:
        super().__init__(config)
        self.num_labels = config.num_labels
        self.transformer = GPT2Model(config)
        p = getattr(config, "classifier_dropout", None)
        if p is None:
            p = getattr(config, "hidden_dropout", None)
        self.dropout = nn.Dropout(0.1 if p is None else p)
        self.classifier = Linear(config.hidden_size, config.num_labels)
        self.post_init()

    def num_blocks(self) -> int:
        return self.transformer.num_blocks()

    def get_head_layers(self) -> List[Layer]:
        c = self.classifier
        return [Layer(module=c, weight=c.weight, bias=c.bias, parallel=False)]

    def head_fn(self, **kw):
        kw["logits"] = self.classifier(self.dropout(kw["hidden_states"]))
        return kw

    def loss_fn(self, **kw):
        kw["loss"] = None
        labels = kw.get("labels")
        if labels is not None:
            logits = kw["logits"]
            am = kw.get("attention_mask")
            if am is not None:
                labels = torch.where(am.view(-1) == 1, labels.view(-1), torch.full_like(labels.view(-1), -100))
            kw["loss"] = F.cross_entropy(logits.view(-1, self.num_labels).float(), labels.view(-1))
        return kw

    def organize_fn(self, **kw):
        out = TokenClassifierOutput(
            loss=kw.get("loss"), logits=kw.get("logits"),
            hidden_states=tuple(kw["all_hidden_states"]) if kw["all_hidden_states"] is not None else None,
            attentions=tuple(kw["all_attentions"]) if kw["all_attentions"] is not None else None)
        return out if kw["return_dict"] else out.to_tuple()

    def forward(self, input_ids=None, **kw):
        kw.setdefault("use_cache", False)
        return self.run_protocol(input_ids=input_ids, **kw)


class GPT2LayerPolicy(LayerPolicy):
    @staticmethod
    def reduce_arguments(layer, world_size, config):
        for a in [layer.attn] + ([layer.crossattention] if hasattr(layer, "crossattention") else []):
            a.embed_dim = config.n_embd // world_size
            a.split_size = config.n_embd // world_size
            a.num_heads = config.n_head // world_size

    @staticmethod
    def fused_modules():
        return {GPT2Attention: FusedGPT2Attention, GPT2MLP: FusedGPT2MLP}

    @staticmethod
    def attn_qkv(layer, config):
        m = layer.attn.c_attn
        out = [Layer(module=m, weight=m.weight, bias=m.bias, n_fused=3, reversed=True, replace={Conv1D: "column"})]
        if hasattr(layer, "crossattention"):
            c = layer.crossattention
            out.append(Layer(module=c.c_attn, weight=c.c_attn.weight, bias=c.c_attn.bias, n_fused=2, reversed=True,
                             replace={Conv1D: "column"}))
            out.append(Layer(module=c.q_attn, weight=c.q_attn.weight, bias=c.q_attn.bias, reversed=True,
                             replace={Conv1D: "column"}))
        return out

    @staticmethod
    def attn_out(layer, config):
        mods = [layer.attn.c_proj] + ([layer.crossattention.c_proj] if hasattr(layer, "crossattention") else [])
        return [Layer(module=m, weight=m.weight, bias=m.bias, reversed=True, replace={Conv1D: "row"}) for m in mods]

    @staticmethod
    def attn_norm(layer, config):
        norms = [layer.ln_1] + ([layer.ln_cross_attn] if hasattr(layer, "ln_cross_attn") else [])
        return [Layer(module=n, weight=n.weight, bias=n.bias, parallel=False) for n in norms]

    @staticmethod
    def mlp_in(layer, config):
        m = layer.mlp.c_fc
        return [Layer(module=m, weight=m.weight, bias=m.bias, reversed=True, replace={Conv1D: "column"})]

    @staticmethod
    def mlp_out(layer, config):
        m = layer.mlp.c_proj
        return [Layer(module=m, weight=m.weight, bias=m.bias, reversed=True, replace={Conv1D: "row"})]

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
        return GPT2Block
