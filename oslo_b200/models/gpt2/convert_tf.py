"""Load an original TensorFlow GPT-2 checkpoint (``model.ckpt`` of the OpenAI release) into a GPT-2 model.

Counterpart of the reference's ``load_tf_weights_in_gpt2`` (oslo/models/gpt2/modeling_gpt2.py:74-128). TensorFlow is
only needed to READ the checkpoint (``tf.train.list_variables`` / ``tf.train.load_variable``); the variable names are
translated to state-dict keys by a pure function, so the mapping itself is testable without TensorFlow:

    model/wte                    -> transformer.wte.weight
    model/h3/attn/c_attn/w       -> transformer.h.3.attn.c_attn.weight      (stored [1, in, out]; squeezed)
    model/h3/ln_1/g, .../b       -> transformer.h.3.ln_1.weight, .bias
    model/ln_f/g                 -> transformer.ln_f.weight
"""
from __future__ import annotations

import logging
import os
import re
from typing import Dict, Optional

import numpy as np
import torch

logger = logging.getLogger(__name__)
_LEAF = {"w": "weight", "g": "weight", "b": "bias"}


def tf_name_to_key(name: str, prefix: str = "transformer.") -> Optional[str]:
    """State-dict key of a TensorFlow variable name, or ``None`` for variables that are not model weights
    (optimizer slots, the global step)."""
    if not name.startswith("model/"):
        return None
    parts = name[len("model/"):].split("/")
    out = []
    for i, part in enumerate(parts):
        last = i == len(parts) - 1
        m = re.fullmatch(r"([A-Za-z_]+?)(\d+)", part)
        if part in ("wte", "wpe") and last:
            out += [part, "weight"]
        elif last and part in _LEAF:
            out.append(_LEAF[part])
        elif m and m.group(1) == "h":
            out += ["h", m.group(2)]
        else:
            out.append(part)
    if out[-1] not in ("weight", "bias"):
        return None
    return prefix + ".".join(out)


def load_tf_weights_in_gpt2(model, config, gpt2_checkpoint_path: str):
    """Fill ``model`` (a ``GPT2Model`` or one of the head models) from a TensorFlow checkpoint; returns the model."""
    try:
        import tensorflow as tf
    except ImportError:
        logger.error("reading a TensorFlow checkpoint needs TensorFlow: https://www.tensorflow.org/install/")
        raise
    tf_path = os.path.abspath(gpt2_checkpoint_path)
    has_prefix = any(k.startswith("transformer.") for k in model.state_dict())
    params: Dict[str, torch.Tensor] = dict(model.named_parameters())
    loaded = 0
    for name, _shape in tf.train.list_variables(tf_path):
        key = tf_name_to_key(name, "transformer." if has_prefix else "")
        if key is None:
            continue
        if key not in params:
            raise KeyError(f"TensorFlow variable {name!r} has no counterpart {key!r} in {type(model).__name__}")
        array = np.asarray(tf.train.load_variable(tf_path, name)).squeeze()
        target = params[key]
        if tuple(target.shape) != tuple(array.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(array.shape)} does not match {key} {tuple(target.shape)}")
        with torch.no_grad():
            target.copy_(torch.from_numpy(np.ascontiguousarray(array)).to(target.dtype))
        loaded += 1
    if hasattr(model, "tie_weights"):
        model.tie_weights()
    logger.info("loaded %d tensors from %s", loaded, tf_path)
    return model
