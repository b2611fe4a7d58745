"""Export description of GPT-2 for ONNX: named inputs / outputs with their dynamic axes and matching dummy inputs.

Counterpart of the reference's ``GPT2OnnxConfig`` (oslo/models/gpt2/configuration_gpt2.py:191-262), which derives
from ``transformers.onnx.OnnxConfigWithPast``; that base class is gone from current transformers releases, so this one
stands alone and keeps the same properties: ``inputs``, ``outputs``, ``generate_dummy_inputs``, ``default_onnx_opset``.
``export()`` drives ``torch.onnx.export`` with them.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Mapping, Optional

import torch


class GPT2OnnxConfig:
    default_onnx_opset = 13
    # names of the config fields that hold the layer count, the head count and the hidden size (sub-classes for other
    # decoder families only change these)
    _layers_attr, _heads_attr, _hidden_attr = "n_layer", "n_head", "n_embd"

    def __init__(self, config, task: str = "default", use_past: bool = False) -> None:
        self._config = config
        self.task = task
        self.use_past = bool(use_past)

    @classmethod
    def with_past(cls, config, task: str = "default") -> "GPT2OnnxConfig":
        return cls(config, task=task, use_past=True)

    @property
    def num_layers(self) -> int:
        return getattr(self._config, self._layers_attr)

    @property
    def num_attention_heads(self) -> int:
        return getattr(self._config, self._heads_attr)

    @property
    def inputs(self) -> Mapping[str, Mapping[int, str]]:
        common = OrderedDict({"input_ids": {0: "batch", 1: "sequence"}})
        if self.use_past:
            for i in range(self.num_layers):
                common[f"past_key_values.{i}.key"] = {0: "batch", 2: "past_sequence"}
                common[f"past_key_values.{i}.value"] = {0: "batch", 2: "past_sequence"}
            common["attention_mask"] = {0: "batch", 1: "past_sequence + sequence"}
        else:
            common["attention_mask"] = {0: "batch", 1: "sequence"}
        return common

    @property
    def outputs(self) -> Mapping[str, Mapping[int, str]]:
        name = "logits" if self.task in ("causal-lm", "causal-lm-with-past") else "last_hidden_state"
        common = OrderedDict({name: {0: "batch", 1: "sequence"}})
        if self.use_past:
            for i in range(self.num_layers):
                common[f"present.{i}.key"] = {0: "batch", 2: "past_sequence + sequence"}
                common[f"present.{i}.value"] = {0: "batch", 2: "past_sequence + sequence"}
        return common

    def generate_dummy_inputs(self, tokenizer=None, batch_size: int = -1, seq_length: int = -1, is_pair: bool = False,
                              framework: Optional[str] = None) -> Mapping[str, Any]:
        """Inputs in the order of ``forward()``: ids, (past key / value pairs), attention mask. Fixed sizes stand in
        for dynamic axes (-1): batch 2, sequence 8. ``tokenizer`` is accepted for call compatibility and unused
        (ids are drawn below the vocabulary size)."""
        batch = 2 if batch_size in (-1, None) else int(batch_size)
        seq = 8 if seq_length in (-1, None) else int(seq_length)
        g = torch.Generator().manual_seed(0)
        ordered = OrderedDict({"input_ids": torch.randint(0, self._config.vocab_size, (batch, seq), generator=g)})
        past = 0
        if self.use_past:
            past = seq + 2       # a past length that differs from the sequence length, so the two axes cannot be confused
            head_dim = getattr(self._config, self._hidden_attr) // self.num_attention_heads
            shape = (batch, self.num_attention_heads, past, head_dim)
            ordered["past_key_values"] = [(torch.zeros(shape), torch.zeros(shape)) for _ in range(self.num_layers)]
        ordered["attention_mask"] = torch.ones(batch, past + seq, dtype=torch.long)
        return ordered

    def export(self, model, path: str, opset: Optional[int] = None) -> str:
        """``torch.onnx.export`` of ``model`` (eval mode, no cache outputs unless ``use_past``) to ``path``."""
        dummy = self.generate_dummy_inputs()
        model = model.eval()
        axes = {k: v for k, v in list(self.inputs.items()) + list(self.outputs.items())}

        class _Wrapper(torch.nn.Module):
            def __init__(self, inner, use_past):
                super().__init__()
                self.inner, self.use_past = inner, use_past

            def forward(self, input_ids, attention_mask):
                out = self.inner(input_ids=input_ids, attention_mask=attention_mask, use_cache=False, return_dict=True)
                return out.logits if getattr(out, "logits", None) is not None else out.last_hidden_state

        if self.use_past:
            raise NotImplementedError("export with past key / values: feed the cache through a wrapper of your own")
        torch.onnx.export(_Wrapper(model, False), (dummy["input_ids"], dummy["attention_mask"]), path,
                          input_names=["input_ids", "attention_mask"], output_names=list(self.outputs),
                          dynamic_axes={k: axes[k] for k in ["input_ids", "attention_mask"] + list(self.outputs)},
                          opset_version=opset or self.default_onnx_opset)
        return path
