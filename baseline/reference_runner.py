"""Reference arm of ``bench.py``: trains the unmodified reference package installed under ``baseline/_ref``
(``oslo`` 2.0.2) through its own public API - ``GPTJForCausalLM.from_config_with_parallel`` for the model,
``model.gpu_modules()`` / ``model.gpu_parameters()`` / ``model.mpu.get_data_parallel_group()`` with torch's
``DistributedDataParallel`` and a torch optimizer for data parallelism, exactly the recipe of the reference's
USAGE.md ("Data Parallelism") - or reports why that is impossible on this stack.

Nothing of ``oslo_b200`` is imported here. The reference was written against transformers 4.x and NumPy 1.x;
``install_compat()`` makes ``import oslo`` possible on the installed versions WITHOUT touching a file of the
reference:

* module aliases: names that moved (``transformers.generation_logits_process`` ->
  ``transformers.generation.logits_process``, ``transformers.modeling_utils.Conv1D`` ->
  ``transformers.pytorch_utils.Conv1D``, ``transformers.file_utils.ModelOutput`` -> ``transformers.utils`` ...)
  resolve to the same objects at their new home;
* names that no longer exist anywhere (beam scorers, ONNX config, ``dacite``: all used by the reference's
  generation / deployment / export code only) resolve to placeholders that raise when instantiated, so the
  training path cannot silently use a stand-in;
* ``PreTrainedModel.init_weights()`` (how 4.x models finish ``__init__``) forwards to 5.x ``post_init()``, and
  ``get_head_mask(None, n)`` returns ``[None] * n`` as it did in 4.x (a head mask that is not None raises).

The training step is the reference's own model code in eager PyTorch; only the measurement harness is ours.
"""
from __future__ import annotations

import contextlib
import importlib
import json
import os
import sys
import time
import types
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

# GPT-J-6B (the reference's `gptj` family at the size of the headline benchmark)
MODELS = {
    "gptj-6b": dict(n_layer=28, n_embd=4096, n_head=16, rotary_dim=64, vocab_size=50400, n_positions=2048),
    "gptj-small": dict(n_layer=4, n_embd=1024, n_head=8, rotary_dim=64, vocab_size=50400, n_positions=2048),
    "gptj-tiny": dict(n_layer=2, n_embd=64, n_head=4, rotary_dim=8, vocab_size=128, n_positions=64),
}

_LEGACY_MODULES = ["transformers.generation_logits_process", "transformers.generation_stopping_criteria",
                   "transformers.generation_utils", "transformers.generation_beam_search", "transformers.file_utils",
                   "transformers.onnx", "transformers.utils.model_parallel_utils", "dacite"]
_NEW_HOMES = ["transformers.generation.logits_process", "transformers.generation.stopping_criteria",
              "transformers.generation.utils", "transformers.generation.beam_search", "transformers.generation",
              "transformers.pytorch_utils", "transformers.modeling_utils", "transformers.utils",
              "transformers.utils.hub", "transformers"]
PLACEHOLDERS: List[str] = []


def _lookup(name: str):
    for mod_name in _NEW_HOMES:
        try:
            mod = importlib.import_module(mod_name)
        except Exception:
            continue
        try:
            return getattr(mod, name)
        except Exception:
            continue
    return None


def _placeholder(name: str):
    PLACEHOLDERS.append(name)

    def _init(self, *a, **k):
        raise NotImplementedError(f"{name} does not exist in the installed transformers / environment")

    return type(name, (), {"__init__": _init})


class _AliasModule(types.ModuleType):
    """``from legacy_module import X`` -> the object called X at its new home, else a raising placeholder."""

    def __getattr__(self, name: str):
        if name.startswith("__"):
            raise AttributeError(name)
        obj = _lookup(name)
        if obj is None:
            obj = _placeholder(name)
        setattr(self, name, obj)
        return obj


def install_compat() -> None:
    import numpy as np
    if not hasattr(np, "float"):
        np.float = float   # alias removed in NumPy 1.24; the reference uses it as a dtype name
    import transformers
    import transformers.modeling_utils as mu
    for legacy in _LEGACY_MODULES:
        if legacy in sys.modules:
            continue
        try:
            importlib.import_module(legacy)
        except Exception:
            sys.modules[legacy] = _AliasModule(legacy)
    # 4.x stopping criteria answered with ONE bool for the whole batch (the reference's loops do ``if criteria(...)``);
    # the installed version answers per sequence. Same criteria objects, the list reduces their answer.
    sc_mod = sys.modules.get("transformers.generation_stopping_criteria")
    if isinstance(sc_mod, _AliasModule) and "StoppingCriteriaList" not in sc_mod.__dict__:
        new_list = _lookup("StoppingCriteriaList")
        if new_list is not None:
            class StoppingCriteriaList(new_list):  # noqa: D401 - name must match the 4.x class
                def __call__(self, input_ids, scores, **kwargs):
                    done = super().__call__(input_ids, scores, **kwargs)
                    return bool(done.all()) if hasattr(done, "all") else bool(done)

            sc_mod.StoppingCriteriaList = StoppingCriteriaList
    for name in ("Conv1D", "SequenceSummary", "find_pruneable_heads_and_indices", "prune_conv1d_layer",
                 "get_parameter_dtype", "unwrap_model"):
        if not hasattr(mu, name):
            setattr(mu, name, _lookup(name) or _placeholder(name))
    if not hasattr(transformers, "cached_path"):
        transformers.cached_path = _lookup("cached_file") or _placeholder("cached_path")
    base = mu.PreTrainedModel
    if not getattr(base, "_oslo_ref_compat", False):
        orig_init_weights = base.init_weights

        def init_weights(self, *a, **k):
            if "all_tied_weights_keys" not in self.__dict__ and not hasattr(type(self), "all_tied_weights_keys"):
                return self.post_init()
            return orig_init_weights(self, *a, **k)

        base.init_weights = init_weights
        if not hasattr(base, "get_head_mask"):
            def get_head_mask(self, head_mask, num_hidden_layers, is_attention_chunked=False):
                if head_mask is not None:
                    raise NotImplementedError("head_mask is not supported by the installed transformers")
                return [None] * num_hidden_layers

            base.get_head_mask = get_head_mask
        base._oslo_ref_compat = True


def probe() -> str:
    """Empty string when ``import oslo`` works from baseline/_ref (with the compatibility aliases), else why not."""
    if not os.path.isdir(os.path.join(REF, "oslo")):
        return "reference package is not installed under baseline/_ref"
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        install_compat()
        import oslo  # noqa: F401
        return ""
    except BaseException as e:  # noqa: BLE001
        return f"import oslo fails on this stack: {type(e).__name__}: {str(e).splitlines()[0][:160]}"


def _emit(obj) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(obj), flush=True)


def _unavailable(why: str) -> None:
    _emit({"impl": "reference", "unavailable": " ".join(str(why).split())[:300]})


def _fits(torch, dev, extra_bytes: int, fraction: float = 0.85) -> bool:
    if dev.type != "cuda":
        return True
    total = torch.cuda.get_device_properties(dev).total_memory
    return torch.cuda.max_memory_allocated(dev) + extra_bytes < fraction * total


def run_train(args, sampler_cls=None, force_cpu: bool = False) -> dict:
    """The reference's training step at ``args.batch_per_gpu`` x ``args.seq`` tokens per GPU per step: forward /
    backward over micro-batches (gradients reduced by torch DDP during the last one), gradient clipping, AdamW."""
    import torch
    import torch.distributed as dist
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if force_cpu:
        dev = torch.device("cpu")
        if not dist.is_initialized():   # the reference's MPU would ask for NCCL; it keeps an existing group
            dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if not dist.is_initialized():   # as under any launcher; the reference's MPU then only creates its groups
            dist.init_process_group("nccl", rank=rank, world_size=world)

    import oslo
    from torch.nn.parallel import DistributedDataParallel
    dims = MODELS[args.model]
    tp, pp = int(getattr(args, "tp", None) or 1), int(getattr(args, "pp", None) or 1)
    if world % (tp * pp):
        raise RuntimeError(f"{world} GPUs cannot be cut into tp={tp} x pp={pp}")
    seq = args.seq
    per_gpu = int(getattr(args, "replica_batch", None) or args.batch_per_gpu * tp * pp)   # sequences per model replica
    cfg = oslo.GPTJConfig(use_cache=False, **dims)
    # model-parallel layouts: no memory probe (a rank that runs out of memory in the middle of a tensor-parallel
    # collective would leave its peers waiting); 2 sequences per tensor-parallel GPU is what the probe settles on
    # for one GPU, and a pipeline stage holds a quarter of the layers
    fixed_micro = None
    if tp * pp > 1:
        fixed_micro = int(getattr(args, "micro_batch", None) or (4 if pp > 1 else 2 * tp))
        fixed_micro = max(1, min(fixed_micro, per_gpu))
        while per_gpu % fixed_micro:
            fixed_micro -= 1

    def build():
        return oslo.GPTJForCausalLM.from_config_with_parallel(
            cfg, tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=fixed_micro or 1,
            torch_dtype=torch.bfloat16)

    try:                                # parameters created on the device (28 x 200 M values: minutes on the host)
        with torch.device(dev):
            model = build()
        init = "on device"
    except Exception:
        model = build()
        init = "on host"
    model = model.to(dev).train()
    mpu = model.mpu
    dp = mpu.get_data_parallel_world_size()
    params = list(model.gpu_parameters())
    opt = torch.optim.AdamW(params, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    param_bytes = sum(p.numel() * p.element_size() for p in params)

    gen = torch.Generator().manual_seed(1000 + mpu.get_data_parallel_rank())
    n_host = 4
    host = [torch.randint(0, dims["vocab_size"], (per_gpu, seq), generator=gen) for _ in range(n_host)]
    if dev.type == "cuda":
        host = [h.pin_memory() for h in host]
    dev_inputs = [h.to(dev) for h in host]

    engine = model      # wrapped in DistributedDataParallel below, after the memory probe

    def fwd_bwd(ids, micro, sync_last=True):
        accum = per_gpu // micro
        total = None
        if pp > 1:
            # the reference's pipeline engine: a generator with one output per micro-batch, backward inside the loop
            # (oslo/parallelism/engine_pipeline.py:262-303)
            for out in engine(input_ids=ids, labels=ids):
                (out.loss / accum).backward()
                total = out.loss.detach().float() if total is None else total + out.loss.detach().float()
            return total / accum
        for i in range(accum):
            mb = ids[i * micro:(i + 1) * micro]
            hold = engine.no_sync() if (dp > 1 and (i < accum - 1 or not sync_last)) else contextlib.nullcontext()
            with hold:
                loss = engine(input_ids=mb, labels=mb).loss
                (loss / accum).backward()
            total = loss.detach().float() if total is None else total + loss.detach().float()
        return total / accum

    # largest micro-batch whose forward/backward leaves room for the optimizer state (the model materialises the
    # attention matrix, so activation memory grows quickly with it); probed without collectives, then agreed
    micro = fixed_micro or 1
    for cand in ([] if fixed_micro else [m for m in (4, 2, 1) if m <= per_gpu and per_gpu % m == 0]):
        ok = True
        try:
            if dev.type == "cuda":
                torch.cuda.reset_peak_memory_stats(dev)
            ids = dev_inputs[0][:cand]
            model(input_ids=ids, labels=ids).loss.backward()   # the bare model: no collective can be left half done
            # still to come: two moments + the multi-tensor update's temporaries, and DDP's gradient buckets
            ok = _fits(torch, dev, (4 + (1 if dp > 1 else 0)) * param_bytes)
        except RuntimeError as e:                     # torch.OutOfMemoryError is a RuntimeError
            if not isinstance(e, torch.OutOfMemoryError) and "out of memory" not in str(e).lower():
                raise
            ok = False
        opt.zero_grad(set_to_none=True)
        if dev.type == "cuda":
            torch.cuda.empty_cache()
        if ok:
            micro = cand
            break
    if dp > 1:
        t = torch.tensor([micro], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        micro = int(t.item())
        kw = dict(device_ids=[local], output_device=local) if dev.type == "cuda" else {}
        engine = DistributedDataParallel(model.gpu_modules(), process_group=mpu.get_data_parallel_group(), **kw)

    def train_step(ids):
        opt.zero_grad(set_to_none=True)
        loss = fwd_bwd(ids, micro)
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        return loss

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize()

    def timed(steps, e2e):
        dist.barrier()
        sync()
        sampler = sampler_cls(local) if (sampler_cls is not None and dev.type == "cuda") else None
        if sampler is not None:
            sampler.start()
        if dev.type == "cuda":
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
        wall0 = time.perf_counter()
        last = None
        for s in range(steps):
            if e2e:
                ids = host[s % n_host].to(dev, non_blocking=True)
                last = float(train_step(ids).item())
            else:
                last = train_step(dev_inputs[s % n_host])
        if dev.type == "cuda":
            t1.record()
        sync()
        wall = time.perf_counter() - wall0
        dist.barrier()
        clocks = sampler.stop() if sampler is not None else None
        ms = wall * 1e3 if (e2e or dev.type != "cuda") else t0.elapsed_time(t1)
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / steps, clocks, last

    for _ in range(args.warmup):
        train_step(dev_inputs[0])
    ms_step, clocks, _ = timed(args.steps, e2e=False)
    tokens_step = dp * per_gpu * seq
    e2e = None
    if not getattr(args, "no_e2e", False):
        ms_e2e, _, loss_host = timed(args.steps, e2e=True)
        e2e = {"value": tokens_step / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": per_gpu * seq * 8, "d2h_bytes_per_step": 4, "last_loss": loss_host}
    line = {
        "impl": "reference",
        "metric": "GPT-J-6B train tokens/sec" if args.model == "gptj-6b" else f"{args.model} train tokens/sec (debug)",
        "value": tokens_step / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
        "config": {"model": args.model, "global_batch": dp * per_gpu, "seq_len": seq,
                   "parallelism": ("x".join(f"{k}{v}" for k, v in (("tp", tp), ("pp", pp), ("dp", dp)) if v > 1) or "single")
                                  + (" (torch DistributedDataParallel over mpu.get_data_parallel_group())" if dp > 1 else "")
                                  + (" (the reference's tensor / pipeline engines)" if tp * pp > 1 else ""),
                   "micro_batch": micro, "grad_accum": per_gpu // micro,
                   "optimizer": "torch.optim.AdamW on bf16 parameters + clip_grad_norm_",
                   "code_path": "oslo 2.0.2 GPTJForCausalLM.from_config_with_parallel, eager (no fuse())",
                   "weights_initialised": init, "device": dev.type,
                   "l2": "working set per step >> 126 MB L2, no explicit flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": None,
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if dev.type == "cuda" else None,
        "compat_placeholders": len(PLACEHOLDERS),
    }
    dist.barrier()
    return line


_GENERATION_DEFAULTS_4X = dict(
    max_length=20, min_length=0, do_sample=False, early_stopping=False, num_beams=1, num_beam_groups=1,
    diversity_penalty=0.0, temperature=1.0, top_k=50, top_p=1.0, repetition_penalty=1.0, length_penalty=1.0,
    no_repeat_ngram_size=0, encoder_no_repeat_ngram_size=0, bad_words_ids=None, num_return_sequences=1,
    output_scores=False, return_dict_in_generate=False, forced_bos_token_id=None, forced_eos_token_id=None,
    remove_invalid_values=False, fused_no_repeat_ngram_blocking=False, is_encoder_decoder=False,
    pad_token_id=None, bos_token_id=None, eos_token_id=None, decoder_start_token_id=None)


def run_decode(args, sampler_cls=None, force_cpu: bool = False) -> dict:
    """Greedy ``generate()`` of the unmodified reference (its vendored 4.x generation loop,
    oslo/generation_utils.py:1108-1361, HF-style concatenated KV cache), tensor parallel over all GPUs: prompts of
    ``--prompt`` tokens, ``--new-tokens`` new tokens. The per-token decode latency is the difference between a call
    that generates ``new_tokens`` tokens and a call that generates one (prefill + first token), divided by
    ``new_tokens - 1``; both are device-timed, max over ranks."""
    import torch
    import torch.distributed as dist
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if force_cpu:
        dev = torch.device("cpu")
        if not dist.is_initialized():
            dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if not dist.is_initialized():
            dist.init_process_group("nccl", rank=rank, world_size=world)
    import oslo
    dims = MODELS[args.model]
    tp = int(getattr(args, "tp", None) or world)
    cfg = oslo.GPTJConfig(use_cache=True, **dims)
    # generate() of the reference reads its defaults from the model config, where transformers 4.x kept them; the
    # installed transformers moved them to GenerationConfig, so the 4.x default values are set as config attributes
    for k, v in _GENERATION_DEFAULTS_4X.items():
        if not hasattr(cfg, k):
            setattr(cfg, k, v)
    with torch.device(dev):
        model = oslo.GPTJForCausalLM.from_config_with_parallel(cfg, tensor_parallel_size=tp, pipeline_parallel_size=1,
                                                               torch_dtype=torch.bfloat16)
    model = model.to(dev).eval()
    b, prompt, n_new = args.decode_batch, args.prompt, args.new_tokens
    gen = torch.Generator().manual_seed(77)
    host = [torch.randint(0, dims["vocab_size"], (b, prompt), generator=gen) for _ in range(4)]
    if dev.type == "cuda":
        host = [h.pin_memory() for h in host]
    dev_inputs = [h.to(dev) for h in host]

    def generate(ids, new):
        with torch.no_grad():
            return model.generate(input_ids=ids, max_length=prompt + new, min_length=prompt + new, do_sample=False,
                                  num_beams=1, use_cache=True, pad_token_id=0, eos_token_id=None)

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize()

    def timed(steps, new, e2e=False):
        dist.barrier()
        sync()
        sampler = sampler_cls(local) if (sampler_cls is not None and dev.type == "cuda") else None
        if sampler is not None:
            sampler.start()
        if dev.type == "cuda":
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
        wall0 = time.perf_counter()
        for s in range(steps):
            if e2e:
                out = generate(host[s % 4].to(dev, non_blocking=True), new).cpu()
            else:
                out = generate(dev_inputs[s % 4], new)
        if dev.type == "cuda":
            t1.record()
        sync()
        wall = time.perf_counter() - wall0
        dist.barrier()
        clocks = sampler.stop() if sampler is not None else None
        ms = wall * 1e3 if (e2e or dev.type != "cuda") else t0.elapsed_time(t1)
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / steps, clocks, out

    for _ in range(args.warmup):
        generate(dev_inputs[0], n_new)
    ms_call, clocks, out = timed(args.steps, n_new)
    ms_first, _, _ = timed(args.steps, 1)
    assert tuple(out.shape) == (b, prompt + n_new), tuple(out.shape)
    ms_tok = (ms_call - ms_first) / max(n_new - 1, 1)
    e2e = None
    if not getattr(args, "no_e2e", False):
        ms_e2e, _, _ = timed(args.steps, n_new, e2e=True)
        e2e = {"value": ms_e2e / n_new, "unit": "ms/token (whole generate call incl. prefill, host in/out)",
               "ms_per_step": ms_e2e, "h2d_bytes_per_step": b * prompt * 8, "d2h_bytes_per_step": b * (prompt + n_new) * 8}
    line = {
        "impl": "reference",
        "metric": f"GPT-J-6B TP={tp} decode ms/token" if args.model == "gptj-6b" else f"{args.model} TP={tp} decode ms/token (debug)",
        "value": ms_tok, "unit": "ms/token", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_call, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random-init weights",
        "config": {"model": args.model, "global_batch": b, "seq_len": prompt, "new_tokens": n_new,
                   "parallelism": f"tp{tp} (the reference's tensor engine)",
                   "decode": "greedy generate(), concatenated KV cache, eager per-token loop",
                   "prefill_plus_first_token_ms": ms_first, "tokens_per_s": b * 1e3 / ms_tok if ms_tok > 0 else None,
                   "code_path": "oslo 2.0.2 GPTJForCausalLM.from_config_with_parallel(...).generate(), eager (no fuse())",
                   "device": dev.type},
        "clocks": clocks, "e2e": e2e, "gpu_launches": None,
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if dev.type == "cuda" else None,
        "compat_placeholders": len(PLACEHOLDERS),
    }
    dist.barrier()
    return line


def main(args, sampler_cls=None) -> None:
    """Print the reference's JSON line, or ``{"impl": "reference", "unavailable": ...}``; never raises."""
    why = probe()
    if why:
        return _unavailable(why)
    if getattr(args, "mode", "train") == "fusion":
        # its script generates with beam search; the beam scorer and the beam-search logits processors that the
        # reference imports from transformers 4.x exist nowhere in the installed release (they are placeholders
        # that raise when instantiated), and its fuse() compiles its kernels at first use for architectures up to
        # sm_80 only
        return _unavailable("the reference's kernel-fusion benchmark needs transformers 4.x beam search classes "
                            "(BeamSearchScorer and others are gone from the installed release) and a JIT build of "
                            "its CUDA kernels, which cannot target sm_100")
    import threading
    limit = float(os.environ.get("OSLO_B200_REFERENCE_DEADLINE_S", "900"))
    done = threading.Event()

    def give_up():
        # a rank that failed while its peers sit in a collective would keep the whole arm alive until the
        # process-group timeout: answer "unavailable" and leave instead
        if not done.is_set():
            _unavailable(f"reference arm did not finish within {limit:.0f} s (a rank failed or a collective never completed)")
            sys.stdout.flush()
            os._exit(0)

    guard = threading.Timer(limit, give_up)
    guard.daemon = True
    guard.start()
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device visible")
        if getattr(args, "mode", "train") == "decode":
            line = run_decode(args, sampler_cls)
        else:
            line = run_train(args, sampler_cls)
        done.set()
        _emit(line)
    except BaseException as e:  # noqa: BLE001 - the arm must exit 0 with a reason, whatever went wrong
        if isinstance(e, (KeyboardInterrupt, SystemExit)):
            raise
        done.set()
        _unavailable(f"reference {getattr(args, 'mode', 'train')} run failed on this stack: {type(e).__name__}: {e}")
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            # peers may be waiting in a collective that this rank will never join: do not wait for them
            sys.stdout.flush()
            os._exit(0)
    finally:
        done.set()
        guard.cancel()
        with contextlib.suppress(Exception):
            import torch
            import torch.distributed as dist
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            if dist.is_initialized():
                dist.destroy_process_group()
