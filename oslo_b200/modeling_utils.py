"""Configuration, output containers and the model base class.

The on-disk contract is the Hugging Face one (``config.json`` + ``pytorch_model.bin`` with HF
parameter names), so hub checkpoints of ``gpt2`` / ``gpt_neo`` / ``gptj`` load unchanged; the
classes themselves are self-contained and need no ``transformers`` install. ``PreTrainedModel``
combines the base with the parallelisation, kernel-fusion and generation mixins
(reference: oslo/modeling_utils.py:107-121).
"""
from __future__ import annotations

import contextlib
import copy
import json
import os
from collections import OrderedDict
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from .fused_kernels_utils import FusedKernelMixin
from .generation.utils import GenerationMixin
from .parallelism_utils import ParallelizationMixin

CONFIG_NAME = "config.json"
WEIGHTS_NAME = "pytorch_model.bin"
SAFE_WEIGHTS_NAME = "model.safetensors"

_DTYPES = {
    "float32": torch.float32, "float": torch.float32, "float16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "float64": torch.float64,
}


def to_torch_dtype(d) -> Optional[torch.dtype]:
    if d is None or isinstance(d, torch.dtype):
        return d
    return _DTYPES[str(d).replace("torch.", "")]


class PretrainedConfig:
    """Attribute bag serialised as HF ``config.json``."""

    model_type = ""
    attribute_map: Dict[str, str] = {}

    def __init__(self, **kwargs: Any) -> None:
        defaults = dict(
            return_dict=True, output_hidden_states=False, output_attentions=False, use_cache=True,
            torch_dtype=None, tie_word_embeddings=True, architectures=None, bos_token_id=None,
            pad_token_id=None, eos_token_id=None, num_labels=2, max_length=20, min_length=0,
            do_sample=False, early_stopping=False, num_beams=1, num_beam_groups=1, diversity_penalty=0.0,
            temperature=1.0, top_k=50, top_p=1.0, repetition_penalty=1.0, length_penalty=1.0,
            no_repeat_ngram_size=0, num_return_sequences=1, fused_no_repeat_ngram_blocking=False,
        )
        for k, v in defaults.items():
            setattr(self, k, kwargs.pop(k, v))
        if isinstance(self.torch_dtype, str):
            self.torch_dtype = to_torch_dtype(self.torch_dtype)
        kwargs.pop("model_type", None)
        kwargs.pop("transformers_version", None)
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __getattr__(self, name: str):
        amap = type(self).attribute_map
        if name in amap and amap[name] != name:
            return getattr(self, amap[name])
        raise AttributeError(name)

    def __setattr__(self, name: str, value: Any) -> None:
        amap = type(self).attribute_map
        object.__setattr__(self, amap.get(name, name), value)

    def to_dict(self) -> Dict[str, Any]:
        out = {k: v for k, v in copy.deepcopy(self.__dict__).items()}
        out["model_type"] = self.model_type
        if isinstance(out.get("torch_dtype"), torch.dtype):
            out["torch_dtype"] = str(out["torch_dtype"]).split(".")[1]
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def save_pretrained(self, save_directory: str) -> None:
        os.makedirs(save_directory, exist_ok=True)
        with open(os.path.join(save_directory, CONFIG_NAME), "w", encoding="utf-8") as f:
            f.write(self.to_json_string())

    @classmethod
    def from_dict(cls, d: Dict[str, Any], **kwargs: Any) -> "PretrainedConfig":
        d = dict(d)
        d.update(kwargs)
        return cls(**d)

    @classmethod
    def from_json_file(cls, path: str, **kwargs: Any) -> "PretrainedConfig":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), **kwargs)

    @classmethod
    def from_pretrained(cls, name_or_path: str, **kwargs: Any) -> "PretrainedConfig":
        path = name_or_path
        if os.path.isdir(path):
            path = os.path.join(path, CONFIG_NAME)
        if not os.path.isfile(path):
            path = _resolve_hub_file(name_or_path, CONFIG_NAME)
        return cls.from_json_file(path, **kwargs)

    def __repr__(self) -> str:
        return f"{type(self).__name__} {self.to_json_string()}"


def _resolve_hub_file(name: str, filename: str) -> str:
    """Find ``filename`` of a hub model id in the local HF cache (no network access is attempted)."""
    try:
        from huggingface_hub import hf_hub_download
        return hf_hub_download(name, filename, local_files_only=True)
    except Exception as e:  # noqa: BLE001
        raise FileNotFoundError(f"cannot find {filename} for {name!r} locally: {e}") from e


class ModelOutput(OrderedDict):
    """Ordered dict with attribute access; ``None`` fields are dropped from tuple/index views."""

    _fields: tuple = ()

    def __init__(self, **kwargs: Any) -> None:
        super().__init__()
        for f in self._fields:
            object.__setattr__(self, f, None)
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __setattr__(self, name: str, value: Any) -> None:
        object.__setattr__(self, name, value)
        if value is not None:
            super().__setitem__(name, value)
        elif name in self:
            super().__delitem__(name)

    def __setitem__(self, key, value) -> None:
        self.__setattr__(key, value)

    def __getitem__(self, k):
        if isinstance(k, str):
            return super().__getitem__(k)
        return self.to_tuple()[k]

    def to_tuple(self) -> tuple:
        return tuple(self[k] for k in self.keys())

    def __reduce__(self):
        return (_rebuild_output, (type(self), dict(self)))


def _rebuild_output(cls, d):
    return cls(**d)


class BaseModelOutputWithPast(ModelOutput):
    _fields = ("last_hidden_state", "past_key_values", "hidden_states", "attentions")


class BaseModelOutputWithPastAndCrossAttentions(ModelOutput):
    _fields = ("last_hidden_state", "past_key_values", "hidden_states", "attentions", "cross_attentions")


class CausalLMOutputWithPast(ModelOutput):
    _fields = ("loss", "logits", "past_key_values", "hidden_states", "attentions")


class CausalLMOutputWithCrossAttentions(ModelOutput):
    _fields = ("loss", "logits", "past_key_values", "hidden_states", "attentions", "cross_attentions")


class SequenceClassifierOutputWithPast(ModelOutput):
    _fields = ("loss", "logits", "past_key_values", "hidden_states", "attentions")


class TokenClassifierOutput(ModelOutput):
    _fields = ("loss", "logits", "hidden_states", "attentions")


class GPT2DoubleHeadsModelOutput(ModelOutput):
    _fields = ("loss", "mc_loss", "logits", "mc_logits", "past_key_values", "hidden_states", "attentions")


class PreTrainedModel(nn.Module, ParallelizationMixin, FusedKernelMixin, GenerationMixin):
    config_class = PretrainedConfig
    base_model_prefix = "transformer"
    is_parallelizable = True
    is_fusable = True
    supports_gradient_checkpointing = True
    _keys_to_ignore_on_save: Optional[List[str]] = None
    _keys_to_ignore_on_load_missing: Optional[List[str]] = None

    def __init__(self, config: PretrainedConfig) -> None:
        super().__init__()
        self.config = config
        self.gradient_checkpointing = False

    # ------------------------------------------------------------------ structure
    @property
    def base_model(self) -> nn.Module:
        return getattr(self, self.base_model_prefix, self)

    @property
    def device(self) -> torch.device:
        for p in self.parameters():
            if p.device.type != "meta":
                return p.device
        return torch.device("cpu")

    @property
    def dtype(self) -> torch.dtype:
        for p in self.parameters():
            if p.is_floating_point():
                return p.dtype
        return torch.float32

    def num_parameters(self, only_trainable: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)

    def get_input_embeddings(self) -> Optional[nn.Module]:
        base = self.base_model
        return base.get_input_embeddings() if base is not self else None

    def set_input_embeddings(self, value: nn.Module) -> None:
        base = self.base_model
        if base is not self:
            base.set_input_embeddings(value)

    def get_output_embeddings(self) -> Optional[nn.Module]:
        return None

    _skip_weight_init = False   # set by `no_weight_init()` while a checkpoint is about to overwrite every tensor

    def post_init(self) -> None:
        if not PreTrainedModel._skip_weight_init:
            self.apply(self._init_weights)
        self.tie_weights()

    def _init_weights(self, module: nn.Module) -> None:
        std = getattr(self.config, "initializer_range", 0.02)
        if isinstance(module, nn.Linear):
            module.weight.data.normal_(mean=0.0, std=std)
            if module.bias is not None:
                module.bias.data.zero_()
        elif isinstance(module, nn.Embedding):
            module.weight.data.normal_(mean=0.0, std=std)
        elif isinstance(module, nn.LayerNorm):
            module.bias.data.zero_()
            module.weight.data.fill_(1.0)
        elif type(module).__name__ == "Conv1D":
            module.weight.data.normal_(mean=0.0, std=std)
            module.bias.data.zero_()

    def tie_weights(self) -> None:
        out, inp = self.get_output_embeddings(), self.get_input_embeddings()
        if out is not None and inp is not None and getattr(self.config, "tie_word_embeddings", True):
            out.weight = inp.weight
            inp.weight._oslo_shared = True   # two layers add into this gradient: no in-place weight-gradient GEMM

    def resize_token_embeddings(self, new_num_tokens: Optional[int] = None) -> nn.Module:
        """Grow/shrink the vocabulary. Only legal before tensor-parallel slicing.

        Reference: oslo/modeling_utils.py:113-121 forbids it on a tensor-parallel model.
        """
        if self.is_tensor_parallelized():
            raise RuntimeError(
                "resize_token_embeddings() cannot run on a tensor-parallel model; pass "
                "`resize_token_embeddings=N` to from_pretrained_with_parallel instead")
        emb = self.get_input_embeddings()
        if new_num_tokens is None or new_num_tokens == emb.num_embeddings:
            return emb
        old = emb.weight.data
        new = old.new_empty(new_num_tokens, old.size(1)).normal_(0.0, getattr(self.config, "initializer_range", 0.02))
        n = min(new_num_tokens, old.size(0))
        new[:n] = old[:n]
        emb.weight = nn.Parameter(new)
        emb.num_embeddings = new_num_tokens
        head = self.get_output_embeddings()
        if head is not None and not getattr(self.config, "tie_word_embeddings", True):
            w = head.weight.data
            nw = w.new_empty(new_num_tokens, w.size(1)).normal_(0.0, 0.02)
            nw[:n] = w[:n]
            head.weight = nn.Parameter(nw)
            if getattr(head, "bias", None) is not None:
                nb = head.bias.data.new_zeros(new_num_tokens)
                nb[:n] = head.bias.data[:n]
                head.bias = nn.Parameter(nb)
            head.out_features = new_num_tokens
        self.config.vocab_size = new_num_tokens
        self.tie_weights()
        return self.get_input_embeddings()

    def gradient_checkpointing_enable(self) -> None:
        for m in self.modules():
            if hasattr(m, "gradient_checkpointing"):
                m.gradient_checkpointing = True

    def gradient_checkpointing_disable(self) -> None:
        for m in self.modules():
            if hasattr(m, "gradient_checkpointing"):
                m.gradient_checkpointing = False

    # ------------------------------------------------------------------ construction / IO
    @classmethod
    def _from_config(cls, config: PretrainedConfig, torch_dtype=None, **kwargs: Any) -> "PreTrainedModel":
        torch_dtype = to_torch_dtype(torch_dtype)
        prev = torch.get_default_dtype()
        if torch_dtype is not None and torch_dtype.is_floating_point:
            torch.set_default_dtype(torch_dtype)
        try:
            model = cls(config, **kwargs)
        finally:
            torch.set_default_dtype(prev)
        return model

    @classmethod
    def from_config(cls, config: PretrainedConfig, **kwargs: Any) -> "PreTrainedModel":
        return cls._from_config(config, **kwargs)

    @classmethod
    def from_pretrained(cls, name_or_path: str, *model_args: Any, config: Optional[PretrainedConfig] = None,
                        state_dict: Optional[Dict[str, torch.Tensor]] = None, torch_dtype=None,
                        low_cpu_mem_usage: bool = False, **kwargs: Any) -> "PreTrainedModel":
        """Load ``config.json`` + ``pytorch_model.bin`` / ``model.safetensors`` from a directory (or the
        local HF cache for a hub id). Unknown kwargs become config attributes, as in HF."""
        if config is None:
            config = cls.config_class.from_pretrained(name_or_path)
        for k in list(kwargs):
            if hasattr(config, k) or not k.startswith("_"):
                setattr(config, k, kwargs.pop(k))
        torch_dtype = to_torch_dtype(torch_dtype)
        if torch_dtype is not None:
            config.torch_dtype = torch_dtype
        if state_dict is None:
            state_dict = load_checkpoint_file(name_or_path)
        if low_cpu_mem_usage:
            # reference: oslo/parallelism_utils.py:345-351. Random initialisation of tensors that the checkpoint
            # overwrites anyway is the slow part of loading a multi-billion-parameter model on the host: skip it,
            # then initialise only what the checkpoint did not bring (e.g. a new classification head)
            with no_weight_init():
                model = cls._from_config(config, torch_dtype=torch_dtype)
            missing = set(model.load_checkpoint_state(state_dict))
            state_dict.clear()
            for name, module in model.named_modules():
                own = [f"{name}.{n}" if name else n for n, _ in module.named_parameters(recurse=False)]
                if any(k in missing for k in own):
                    model._init_weights(module)
        else:
            model = cls._from_config(config, torch_dtype=torch_dtype)
            model.load_checkpoint_state(state_dict)
        model.tie_weights()
        model.eval()
        return model

    def load_checkpoint_state(self, state_dict: Dict[str, torch.Tensor], strict: bool = False):
        """``load_state_dict`` that tolerates the base-model prefix being present or absent and
        drops legacy buffers (``attn.bias`` / ``attn.masked_bias``) found in old HF files."""
        own = self.state_dict()
        prefix = self.base_model_prefix + "."
        has_prefix_model = any(k.startswith(prefix) for k in own)
        has_prefix_ckpt = any(k.startswith(prefix) for k in state_dict)
        fixed = {}
        for k, v in state_dict.items():
            if has_prefix_model and not has_prefix_ckpt and (prefix + k) in own:
                k = prefix + k
            elif not has_prefix_model and has_prefix_ckpt and k.startswith(prefix):
                k = k[len(prefix):]
            if k in own:
                fixed[k] = v
        missing = [k for k in own if k not in fixed]
        ignore = self._keys_to_ignore_on_load_missing or []
        hard_missing = [k for k in missing if not any(pat in k for pat in ignore) and not _is_tied_key(self, k)]
        if strict and hard_missing:
            raise KeyError(f"missing keys: {hard_missing}")
        self.load_state_dict(fixed, strict=False)
        return hard_missing

    def save_pretrained(self, save_directory: str, save_config: bool = True,
                        state_dict: Optional[Dict[str, torch.Tensor]] = None, save_function=torch.save,
                        **kwargs: Any) -> None:
        os.makedirs(save_directory, exist_ok=True)
        if save_config:
            self.config.torch_dtype = self.dtype
            self.config.architectures = [type(self).__name__]
            self.config.save_pretrained(save_directory)
        if state_dict is None:
            state_dict = self.state_dict()
        ignore = self._keys_to_ignore_on_save or []
        state_dict = {k: v for k, v in state_dict.items() if k not in ignore}
        from .utils.checkpoint import atomic_save
        atomic_save(state_dict, os.path.join(save_directory, WEIGHTS_NAME), save_function)


@contextlib.contextmanager
def no_weight_init():
    """Build modules without filling their parameters: ``torch.nn.init``'s random fills (what ``nn.Linear`` /
    ``nn.Embedding`` run in their constructors) and ``PreTrainedModel.post_init``'s pass become no-ops."""
    import torch.nn.init as init
    names = ("kaiming_uniform_", "uniform_", "normal_", "trunc_normal_", "xavier_uniform_", "xavier_normal_")
    saved = {n: getattr(init, n) for n in names}
    prev = PreTrainedModel._skip_weight_init
    try:
        for n in names:
            setattr(init, n, lambda tensor, *a, **k: tensor)
        PreTrainedModel._skip_weight_init = True
        yield
    finally:
        for n, f in saved.items():
            setattr(init, n, f)
        PreTrainedModel._skip_weight_init = prev


def _is_tied_key(model: PreTrainedModel, key: str) -> bool:
    return key.startswith("lm_head.weight") and getattr(model.config, "tie_word_embeddings", True)


def _load_one_file(path: str) -> Dict[str, torch.Tensor]:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    from .utils.checkpoint import load_file as load_checked
    return load_checked(path)      # a truncated / damaged file is reported by name


def _load_sharded(directory: str, index_name: str) -> Dict[str, torch.Tensor]:
    """Hugging Face sharded checkpoint: ``<name>.index.json`` maps every key to one of several shard files
    (how multi-GB checkpoints such as GPT-J-6B are published)."""
    import json
    with open(os.path.join(directory, index_name)) as f:
        weight_map = json.load(f)["weight_map"]
    state: Dict[str, torch.Tensor] = {}
    for shard in sorted(set(weight_map.values())):
        full = os.path.join(directory, shard)
        if not os.path.isfile(full):
            raise FileNotFoundError(f"{index_name} names {shard}, which is missing from {directory!r}")
        state.update(_load_one_file(full))
    missing = [k for k in weight_map if k not in state]
    if missing:
        raise RuntimeError(f"{index_name}: {len(missing)} keys not found in their shard files, e.g. {missing[:3]}")
    return state


def load_checkpoint_file(name_or_path: str) -> Dict[str, torch.Tensor]:
    cands = []
    if os.path.isdir(name_or_path):
        cands = [os.path.join(name_or_path, WEIGHTS_NAME), os.path.join(name_or_path, SAFE_WEIGHTS_NAME)]
        if not any(os.path.isfile(c) for c in cands):
            for index_name in (WEIGHTS_NAME + ".index.json", SAFE_WEIGHTS_NAME + ".index.json"):
                if os.path.isfile(os.path.join(name_or_path, index_name)):
                    return _load_sharded(name_or_path, index_name)
    elif os.path.isfile(name_or_path):
        cands = [name_or_path]
    for c in cands:
        if os.path.isfile(c):
            return _load_one_file(c)
    for fn in (WEIGHTS_NAME, SAFE_WEIGHTS_NAME):
        try:
            return load_checkpoint_file(_resolve_hub_file(name_or_path, fn))
        except FileNotFoundError:
            continue
    raise FileNotFoundError(f"no {WEIGHTS_NAME} or {SAFE_WEIGHTS_NAME} under {name_or_path!r}")
