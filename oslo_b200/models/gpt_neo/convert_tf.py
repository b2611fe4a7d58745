"""Load a mesh-tensorflow GPT-Neo checkpoint (the EleutherAI release) into a GPT-Neo model.

Counterpart of the reference's ``load_tf_weights_in_gpt_neo`` (oslo/models/gpt_neo/modeling_gpt_neo.py:52-146).
TensorFlow is only needed to READ the checkpoint; the translation of variable names is a pure function
(``tf_name_to_key``), testable without TensorFlow:

    gpt2/wte                                   -> transformer.wte.weight     (rows beyond ``vocab_size`` are padding)
    gpt2/h3/attn/q | k | v | o                 -> transformer.h.3.attn.attention.{q,k,v,out}_proj.weight   (transposed)
    gpt2/h3/attn/compute_output_bias/o_b       -> transformer.h.3.attn.attention.out_proj.bias
    gpt2/h3/norm_1/g, norm_2/b                 -> transformer.h.3.ln_1.weight, ln_2.bias
    gpt2/h3/mlp/conv1d_main/c_fc/kernel, bias  -> transformer.h.3.mlp.c_fc.weight (transposed), .bias
    gpt2/ln_f/g                                -> transformer.ln_f.weight
"""
from __future__ import annotations

import logging
import os
import re
from typing import Dict, Optional, Tuple

import numpy as np
import torch

logger = logging.getLogger(__name__)

_ATTN = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "out_proj"}
_NORM = {"norm_1": "ln_1", "norm_2": "ln_2", "ln_f": "ln_f"}


def tf_name_to_key(name: str, prefix: str = "transformer.") -> Optional[Tuple[str, bool]]:
    """``(state-dict key, stored transposed)`` of a checkpoint variable, or ``None`` for variables that are not model
    weights (optimizer slots, the global step)."""
    if "global_step" in name or "adam" in name.lower() or not name.startswith("gpt2/"):
        return None
    parts = name[len("gpt2/"):].split("/")
    if parts in (["wte"], ["wpe"]):
        return prefix + parts[0] + ".weight", False
    out = []
    m = re.fullmatch(r"h(\d+)", parts[0])
    if m:
        out += ["h", m.group(1)]
        parts = parts[1:]
    if not parts:
        return None
    body, leaf = parts[:-1], parts[-1]
    if body == ["attn"] and leaf in _ATTN:
        return prefix + ".".join(out + ["attn", "attention", _ATTN[leaf], "weight"]), True
    if parts == ["attn", "compute_output_bias", "o_b"]:
        return prefix + ".".join(out + ["attn", "attention", "out_proj", "bias"]), False
    if len(body) == 1 and body[0] in _NORM and leaf in ("g", "b"):
        return prefix + ".".join(out + [_NORM[body[0]], "weight" if leaf == "g" else "bias"]), False
    if body[:2] == ["mlp", "conv1d_main"] and len(body) == 3 and body[2] in ("c_fc", "c_proj") \
            and leaf in ("kernel", "bias"):
        return prefix + ".".join(out + ["mlp", body[2], "weight" if leaf == "kernel" else "bias"]), leaf == "kernel"
    return None


def load_tf_weights_in_gpt_neo(model, config, gpt_neo_checkpoint_path: str):
    """Fill ``model`` (a ``GPTNeoModel`` or one of the head models) from a mesh-tensorflow checkpoint; returns it."""
    try:
        import tensorflow as tf
    except ImportError:
        logger.error("reading a TensorFlow checkpoint needs TensorFlow: https://www.tensorflow.org/install/")
        raise
    tf_path = os.path.abspath(gpt_neo_checkpoint_path)
    has_prefix = any(k.startswith("transformer.") for k in model.state_dict())
    params: Dict[str, torch.Tensor] = dict(model.named_parameters())
    loaded = 0
    for name, _shape in tf.train.list_variables(tf_path):
        mapped = tf_name_to_key(name, "transformer." if has_prefix else "")
        if mapped is None:
            continue
        key, transposed = mapped
        if key not in params:
            raise KeyError(f"TensorFlow variable {name!r} has no counterpart {key!r} in {type(model).__name__}")
        array = np.asarray(tf.train.load_variable(tf_path, name), dtype=np.float32).squeeze()
        if transposed:
            array = array.T
        target = params[key]
        if key.endswith("wte.weight"):
            array = array[: target.shape[0]]           # the release pads the vocabulary
        if tuple(target.shape) != tuple(array.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(array.shape)} does not match {key} {tuple(target.shape)}")
        with torch.no_grad():
            target.copy_(torch.from_numpy(np.ascontiguousarray(array)).to(target.dtype))
        loaded += 1
    if hasattr(model, "tie_weights"):
        model.tie_weights()                             # the LM head shares the word embedding
    logger.info("loaded %d tensors from %s", loaded, tf_path)
    return model
