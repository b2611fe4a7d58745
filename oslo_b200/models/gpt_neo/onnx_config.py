"""Export description of GPT-Neo for ONNX: named inputs / outputs with their dynamic axes and dummy inputs.

Counterpart of the reference's ``GPTNeoOnnxConfig`` (oslo/models/gpt_neo/configuration_gpt_neo.py:223-330). The
reference also carries ``custom_unfold`` and ``custom_get_block_length_and_num_blocks`` (:184-220), which patch a
block-wise local attention that slices the sequence with ``Tensor.unfold`` and Python control flow; local layers here
are ordinary attention with a sliding-window mask (a kernel argument on GPUs), so there is nothing to patch for export.
"""
from __future__ import annotations

from ..gpt2.onnx_config import GPT2OnnxConfig


class GPTNeoOnnxConfig(GPT2OnnxConfig):
    _layers_attr, _heads_attr, _hidden_attr = "num_layers", "num_heads", "hidden_size"
