"""``ParallelizationMixin``: the public parallelisation API of every model.

Entry points and checkpoint layout follow the reference (oslo/parallelism_utils.py:375-562):

* ``from_pretrained_with_parallel`` / ``from_config_with_parallel`` / ``oslo_b200.parallelize``
* ``save_pretrained_with_parallel`` writing either one merged HF checkpoint or per-rank files
  ``pytorch_model_tp={i}_pp={j}.bin`` (written by data-parallel rank 0 only)
* ``gpu_modules()`` / ``gpu_parameters()`` for wrapping with DDP / ZeRO style engines
* the six-function forward protocol ``preblock_fn -> block_fn(layer_id) ... -> postblock_fn ->
  head_fn -> loss_fn -> organize_fn`` that the pipeline engine cuts into stages.
"""
from __future__ import annotations

import logging
import os
import random
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)

WEIGHTS_NAME_PARALLEL = "pytorch_model_tp={tp}_pp={pp}.bin"
_PARALLEL_KEYS = ("tensor_parallel_size", "pipeline_parallel_size", "micro_batch_size",
                  "resize_token_embeddings", "seed", "deployment", "sequence_parallel", "pipeline_partition")


def split_checkpoint_names(tp: int, pp: int) -> List[str]:
    return [WEIGHTS_NAME_PARALLEL.format(tp=i, pp=j) for i in range(tp) for j in range(pp)]


def set_seed(seed: Optional[int]) -> None:
    if seed is None:
        return
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class ParallelizationMixin:
    # ------------------------------------------------------------------ model protocol
    def get_layer_policies(self):
        raise NotImplementedError(f"{type(self).__name__} does not define layer policies")

    def get_head_layers(self):
        return []

    def preblock_fn(self, **kw):
        return self.base_model.preblock_fn(**kw)

    def block_fn(self, layer_id: int, **kw):
        return self.base_model.block_fn(layer_id=layer_id, **kw)

    def postblock_fn(self, **kw):
        return self.base_model.postblock_fn(**kw)

    def head_fn(self, **kw):
        return kw

    def loss_fn(self, **kw):
        return kw

    def organize_fn(self, **kw):
        return self.base_model.organize_fn(**kw)

    def num_blocks(self) -> int:
        return len(self.base_model.h)

    def run_protocol(self, **kw):
        """Single-process forward: run the six protocol functions back to back."""
        kw = self.preblock_fn(**kw)
        for i in range(self.num_blocks()):
            kw = self.block_fn(layer_id=i, **kw)
        kw = self.postblock_fn(**kw)
        kw = self.head_fn(**kw)
        kw = self.loss_fn(**kw)
        return self.organize_fn(**kw)

    # ------------------------------------------------------------------ state queries
    @staticmethod
    def make_outputs(kwargs: Dict[str, Any], **outputs: Any) -> Dict[str, Any]:
        """Merge a protocol function's results into the kwargs dict that threads through
        ``preblock_fn -> block_fn -> postblock_fn -> head_fn -> loss_fn -> organize_fn``
        (reference: oslo/parallelism_utils.py:128-131); custom models written against the reference call it."""
        kwargs.update(outputs)
        return kwargs

    def is_model_parallelized(self) -> bool:
        return self.is_tensor_parallelized() or self.is_pipeline_parallelized()

    def is_data_parallelized(self) -> bool:
        mpu = getattr(self, "mpu", None)
        return mpu is not None and mpu.get_data_parallel_world_size() > 1

    def is_tensor_parallelized(self) -> bool:
        mpu = getattr(self, "mpu", None)
        return mpu is not None and mpu.get_tensor_parallel_world_size() > 1

    def is_pipeline_parallelized(self) -> bool:
        mpu = getattr(self, "mpu", None)
        return mpu is not None and mpu.get_pipeline_parallel_world_size() > 1

    def gpu_modules(self):
        """The module to hand to a data-parallel / ZeRO wrapper: this rank's stage under pipeline
        parallelism (its ``forward`` is the pipeline generator), otherwise the model itself."""
        if self.is_pipeline_parallelized():
            return self._pipe_engine.stage_module
        return self

    def gpu_parameters(self):
        return self.gpu_modules().parameters()

    def set_micro_batch_size(self, n: int) -> None:
        eng = getattr(self, "_pipe_engine", None)
        if eng is not None:
            eng.micro_batch_size = int(n)

    # ------------------------------------------------------------------ engines
    def _exec_both_engines(self, tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                           micro_batch_size: int = 1, resize_token_embeddings: Optional[int] = None,
                           seed: Optional[int] = None, sequence_parallel: bool = False,
                           device: Optional[torch.device] = None, pipeline_partition: Optional[List[int]] = None,
                           **_unused: Any):
        from .parallel.engine_pipeline import PipelineParallelEngine
        from .parallel.engine_tensor import TensorParallelEngine
        from .parallel.mpu import MPU

        tp, pp = int(tensor_parallel_size), int(pipeline_parallel_size)
        if tp & (tp - 1):
            raise ValueError(f"tensor_parallel_size must be a power of two, got {tp}")
        if self.is_model_parallelized():
            # slicing sliced weights again would silently corrupt them
            raise RuntimeError("this model is already parallelized; merge it first "
                               "(save_pretrained_with_parallel(..., save_with_merging=True)) to change the layout")
        set_seed(seed)
        if resize_token_embeddings is not None:
            self.resize_token_embeddings(resize_token_embeddings)
        mpu = MPU(tp, pp)
        device = device or mpu.device
        pipe = PipelineParallelEngine(self, mpu, micro_batch_size=micro_batch_size, device=device,
                                      partition=pipeline_partition if pp > 1 else None)
        pipe.assign_stages()
        if tp > 1:
            TensorParallelEngine(self, mpu, owned=pipe.owns_param, device=device,
                                 sequence_parallel=sequence_parallel).parallelize()
        pipe.finalize()
        if pp > 1 and pipe.last and getattr(self.config, "tie_word_embeddings", True) \
                and self.get_output_embeddings() is not None:
            # the last stage's copy of a tied embedding carries the same (summed) gradient as the first stage's
            self.get_input_embeddings().weight._oslo_norm_dup = True
        self.initial_parameters = dict(
            tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=micro_batch_size,
            resize_token_embeddings=resize_token_embeddings, seed=seed, sequence_parallel=sequence_parallel,
            pipeline_partition=list(pipeline_partition) if (pipeline_partition and pp > 1) else None)
        self.mpu = mpu
        if self.base_model is not self:
            self.base_model.mpu = mpu
        return self

    @classmethod
    def _exec_deployment_engine(cls, model, **kwargs):
        from .parallel.engine_deployment import DeploymentParallelEngine
        return DeploymentParallelEngine(model, **kwargs).parallelize()

    @classmethod
    def _parallelize_from_model(cls, model, **kwargs):
        if kwargs.get("deployment"):
            return cls._exec_deployment_engine(model, **kwargs)
        kwargs.pop("deployment", None)
        return model._exec_both_engines(**kwargs)

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_config_with_parallel(cls, config, tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                                  micro_batch_size: int = 1, resize_token_embeddings: Optional[int] = None,
                                  seed: Optional[int] = None, deployment: Optional[bool] = None,
                                  sequence_parallel: bool = False, init_on_device: bool = False,
                                  pipeline_partition: Optional[List[int]] = None, **kwargs: Any):
        """Random-init model from ``config``, then parallelise. ``init_on_device`` builds the full
        model on this rank's accelerator (fast for multi-billion-parameter configs) before slicing.
        ``pipeline_partition``: blocks per pipeline stage, when the even split is not wanted."""
        torch_dtype = kwargs.pop("torch_dtype", getattr(config, "torch_dtype", None))
        for k, v in kwargs.items():
            setattr(config, k, v)
        set_seed(seed)
        if init_on_device and deployment:
            # the deployment workers build the model on their own devices; the parent keeps a weightless handle
            with torch.device("meta"):
                model = cls._from_config(config, torch_dtype=torch_dtype)
            from .parallel.engine_deployment import DeploymentParallelEngine
            return DeploymentParallelEngine(
                model, tensor_parallel_size=tensor_parallel_size, pipeline_parallel_size=pipeline_parallel_size,
                micro_batch_size=micro_batch_size, resize_token_embeddings=resize_token_embeddings, seed=seed,
                sequence_parallel=sequence_parallel, pipeline_partition=pipeline_partition,
                factory=(cls, config, torch_dtype)).parallelize()
        if init_on_device and torch.cuda.is_available() and not deployment:
            from .parallel.mpu import MPU
            MPU.initialize_distributed()
            with torch.device("cuda", torch.cuda.current_device()):
                model = cls._from_config(config, torch_dtype=torch_dtype)
        else:
            model = cls._from_config(config, torch_dtype=torch_dtype)
        return cls._parallelize_from_model(
            model, tensor_parallel_size=tensor_parallel_size, pipeline_parallel_size=pipeline_parallel_size,
            micro_batch_size=micro_batch_size, resize_token_embeddings=resize_token_embeddings, seed=seed,
            deployment=deployment, sequence_parallel=sequence_parallel, pipeline_partition=pipeline_partition)

    @classmethod
    def from_pretrained_with_parallel(cls, pretrained_model_name_or_path: str, tensor_parallel_size: int = 1,
                                      pipeline_parallel_size: int = 1, micro_batch_size: int = 1,
                                      resize_token_embeddings: Optional[int] = None, seed: Optional[int] = None,
                                      deployment: Optional[bool] = None, sequence_parallel: bool = False,
                                      pipeline_partition: Optional[List[int]] = None, **kwargs: Any):
        """Load and parallelise. A directory holding every ``pytorch_model_tp=*_pp=*.bin`` of the
        requested layout is read shard-wise (each rank opens only its own file); anything else is
        loaded as a merged HF checkpoint on the host and sliced."""
        par = dict(tensor_parallel_size=tensor_parallel_size, pipeline_parallel_size=pipeline_parallel_size,
                   micro_batch_size=micro_batch_size, resize_token_embeddings=resize_token_embeddings,
                   seed=seed, deployment=deployment, sequence_parallel=sequence_parallel,
                   pipeline_partition=pipeline_partition)
        path = pretrained_model_name_or_path
        if os.path.isdir(path):
            names = split_checkpoint_names(tensor_parallel_size, pipeline_parallel_size)
            present = [os.path.isfile(os.path.join(path, n)) for n in names]
            any_split = any(f.startswith("pytorch_model_tp=") for f in os.listdir(path))
            if all(present) and any_split:
                return cls._parallelize_from_split_checkpoint_files(path, par, **kwargs)
            if any_split and not os.path.isfile(os.path.join(path, "pytorch_model.bin")):
                missing = [n for n, ok in zip(names, present) if not ok]
                raise FileNotFoundError(
                    f"{path} holds split checkpoints that do not match tensor_parallel_size="
                    f"{tensor_parallel_size}, pipeline_parallel_size={pipeline_parallel_size}; missing {missing}")
        model = cls.from_pretrained(path, **kwargs)
        return cls._parallelize_from_model(model, **par)

    @classmethod
    def _parallelize_from_split_checkpoint_files(cls, path: str, par: Dict[str, Any], **kwargs: Any):
        config = kwargs.pop("config", None) or cls.config_class.from_pretrained(path)
        torch_dtype = kwargs.pop("torch_dtype", getattr(config, "torch_dtype", None))
        low_mem = bool(kwargs.pop("low_cpu_mem_usage", False))
        for k, v in kwargs.items():
            setattr(config, k, v)
        set_seed(par.get("seed"))
        if low_mem:   # every tensor this rank keeps comes from its file: skip the random fill of the full model
            from .modeling_utils import no_weight_init
            with no_weight_init():
                model = cls._from_config(config, torch_dtype=torch_dtype)
        else:
            model = cls._from_config(config, torch_dtype=torch_dtype)
        if par.get("deployment"):
            return cls._exec_deployment_engine(model, split_checkpoint_path=path, **par)
        par = {k: v for k, v in par.items() if k != "deployment"}
        model._exec_both_engines(**par)
        model._load_split_checkpoint_files(path)
        return model

    def _load_split_checkpoint_files(self, path: str) -> None:
        mpu = self.mpu
        fn = WEIGHTS_NAME_PARALLEL.format(tp=mpu.get_tensor_parallel_rank(), pp=mpu.get_pipeline_parallel_rank())
        full = os.path.join(path, fn)
        if not os.path.isfile(full):
            raise FileNotFoundError(full)
        from .utils.checkpoint import load_file
        state = load_file(full)           # names the file if it is truncated or damaged
        own = self.state_dict()
        bad = []
        for k, v in state.items():
            if k not in own or own[k].numel() == 0:
                continue
            if own[k].shape != v.shape:
                bad.append((k, tuple(v.shape), tuple(own[k].shape)))
                continue
            own[k].copy_(v)
        if bad:
            raise RuntimeError(f"split checkpoint {fn} does not match this layout: {bad[:4]}")
        self.tie_weights()
        self._sync_tied_embedding_across_stages()
        self.eval()
        logger.info("loaded %s", full)

    @torch.no_grad()
    def _sync_tied_embedding_across_stages(self) -> None:
        """An output embedding tied to the input embedding lives twice under pipeline parallelism (first and last
        stage). Split files written without the last stage's copy would leave it at its random initialisation, so
        after loading the first stage's tensor is sent to the last stage."""
        mpu, eng = self.mpu, getattr(self, "_pipe_engine", None)
        if eng is None or mpu.get_pipeline_parallel_world_size() == 1 or not (eng.first or eng.last):
            return
        if not getattr(self.config, "tie_word_embeddings", True) or self.get_output_embeddings() is None:
            return
        w = self.get_input_embeddings().weight
        dist.broadcast(w.data, src=mpu.stage_to_global_rank(0), group=mpu.get_embedding_tied_group())

    # ------------------------------------------------------------------ saving
    @torch.no_grad()
    def save_pretrained_with_parallel(self, save_directory: str, save_config: bool = True,
                                      save_with_merging: bool = False, state_dict: Optional[dict] = None,
                                      save_function=torch.save, **kwargs: Any) -> None:
        """Write a checkpoint of a (possibly) parallel model.

        * not parallel: plain ``save_pretrained`` on rank 0.
        * ``save_with_merging=True``: gather tensor-parallel shards and pipeline stages into one HF
          ``pytorch_model.bin`` on rank 0 (the live model is left untouched).
        * otherwise: every (tp, pp) coordinate of data-parallel rank 0 writes its own
          ``pytorch_model_tp={i}_pp={j}.bin``.
        """
        if os.path.isfile(save_directory):
            raise ValueError(f"{save_directory} is a file, expected a directory")
        from .utils.checkpoint import atomic_save      # write beside, then rename: no truncated file after a crash
        os.makedirs(save_directory, exist_ok=True)
        mpu = getattr(self, "mpu", None)
        rank0 = (not dist.is_initialized()) or dist.get_rank() == 0
        if not self.is_model_parallelized():
            if rank0:
                self.save_pretrained(save_directory, save_config=save_config, state_dict=state_dict,
                                     save_function=save_function, **kwargs)
            _barrier()
            return
        if save_with_merging:
            from .parallel.engine_pipeline import PipelineDeparallelEngine
            from .parallel.engine_tensor import TensorDeparallelEngine
            state = state_dict if state_dict is not None else self.state_dict()
            state = PipelineDeparallelEngine(self, mpu).gather_state(state)
            state = TensorDeparallelEngine(self, mpu).merge_state(state)
            if rank0:
                cfg = self._merged_config()
                if save_config:
                    cfg.torch_dtype = self.dtype
                    cfg.architectures = [type(self).__name__]
                    cfg.save_pretrained(save_directory)
                ignore = self._keys_to_ignore_on_save or []
                state = {k: v for k, v in state.items() if k not in ignore}
                atomic_save(state, os.path.join(save_directory, "pytorch_model.bin"), save_function)
            _barrier()
            return
        if save_config and rank0:
            cfg = self._merged_config()
            cfg.torch_dtype = self.dtype
            cfg.architectures = [type(self).__name__]
            cfg.save_pretrained(save_directory)
        state = state_dict if state_dict is not None else self.state_dict()
        ignore = self._keys_to_ignore_on_save or []
        eng = getattr(self, "_pipe_engine", None)
        out = {}
        for k, v in state.items():
            # keys a model leaves out because they are tied to another tensor of the SAME file (GPT-Neo's lm_head);
            # under pipeline parallelism the last stage's copy is the only one in its file, so it stays
            if k in ignore and mpu.get_pipeline_parallel_world_size() == 1:
                continue
            if eng is not None and not eng.owns_key(k):
                continue
            out[k] = v.detach().cpu()
        fn = WEIGHTS_NAME_PARALLEL.format(tp=mpu.get_tensor_parallel_rank(), pp=mpu.get_pipeline_parallel_rank())
        if mpu.get_data_parallel_rank() == 0:
            atomic_save(out, os.path.join(save_directory, fn), save_function)
        _barrier()
        logger.info("saved %s", os.path.join(save_directory, fn))

    # ------------------------------------------------------------------ resume (not in the reference)
    def save_training_state(self, save_directory: str, optimizer=None, step: int = 0, extra=None) -> str:
        """This rank's resume sidecar (optimizer shard, loss scale, step, generators) beside the model files;
        call on every rank. See ``oslo_b200.utils.checkpoint``."""
        from .utils.checkpoint import save_training_state
        return save_training_state(save_directory, optimizer, step, getattr(self, "mpu", None), extra)

    def load_training_state(self, save_directory: str, optimizer=None, restore_rng: bool = True):
        from .utils.checkpoint import load_training_state
        return load_training_state(save_directory, optimizer, getattr(self, "mpu", None), restore_rng)

    def _merged_config(self):
        import copy
        return copy.deepcopy(self.config)


def _barrier() -> None:
    if dist.is_initialized():
        dist.barrier()
