#!/usr/bin/env python
"""Flagship benchmark: GPT-J-6B causal-LM training tokens/s (bf16, AdamW with fp32 master weights).

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run`` for N > 1) prints ONE
JSON line on rank 0. Weak scaling: every GPU works on ``--batch-per-gpu`` sequences of ``--seq`` tokens
per step, so the global batch is ``8 N x 2048`` by default (64 x 2048 on 8 GPUs). Synthetic data: token
ids uniform in [0, vocab) with a fixed seed; weights random-init.

Without ``--tp`` / ``--pp`` the headline follows the model-parallel sweep: one GPU, ``tp2`` on 2 GPUs, ``tp4`` on
4, ``tp2 x pp4`` (16 micro-batches of 4 sequences, 1F1B) on 8; the other named configurations of that GPU count
(ZeRO-1 data parallelism over all GPUs; on 8 GPUs also ``tp8`` with a global batch of 8 x 2048 and GPT-Neo 1.3B as
``tp2 x pp2 x dp2``) are measured in the same invocation and reported under ``"also"``. ``--tp`` / ``--pp`` time exactly one layout.

Timed regions (CUDA events on the compute stream, barrier + synchronize on both sides, max over ranks):
  * ``value``: K full steps (forward, backward, gradient reduction, optimizer) with inputs already on
    the device;
  * ``e2e``: K more steps through the same public API where every step copies its inputs from pinned
    host memory and reads the loss back to the host.
The working set of one step (tens of GB of weights, activations and optimizer state) is far larger
than the 126 MB L2, so no explicit flush is done between iterations (recorded in ``config``).

``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` when it can be
imported on this stack, otherwise prints ``{"impl": "reference", "unavailable": ...}``.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    # name: (n_layer, n_embd, n_head, rotary_dim, vocab, n_positions)
    "gptj-6b": (28, 4096, 16, 64, 50400, 2048),
    "gptj-small": (4, 1024, 8, 64, 50400, 2048),   # debugging only; numbers from it are not benchmark values
    # GPT-Neo 1.3B: alternating global / local (window 256) attention, learned positions; rotary_dim unused
    "gpt-neo-1.3b": (24, 2048, 16, 0, 50257, 2048),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="oslo_b200", choices=["oslo_b200", "reference"])
    ap.add_argument("--model", default="gptj-6b", choices=sorted(MODELS))
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch-per-gpu", type=int, default=8)
    ap.add_argument("--replica-batch", type=int, default=None, help="sequences per model replica per step (default: batch-per-gpu x tp x pp)")
    ap.add_argument("--micro-batch", type=int, default=None, help="sequences per forward/backward (default: auto)")
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--pp", type=int, default=None)
    ap.add_argument("--no-also", action="store_true", help="time the headline configuration only")
    ap.add_argument("--even-partition", action="store_true",
                    help="pipeline parallel: the same number of blocks on every stage (default: the last stage, which "
                         "also runs the LM head and the loss, gets fewer blocks)")
    ap.add_argument("--also-timeout", type=float, default=240.0,
                    help="seconds the extra configurations may take before the headline is printed without them (at "
                         "least; the limit grows to 1.5 x the headline configuration's own run time per extra block)")
    ap.add_argument("--checkpoint-activations", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--mode", default="train", choices=["train", "decode", "fusion"],
                    help="train: tokens/s of a training step; decode: ms/token of greedy generation with a KV cache; "
                         "fusion: seconds of one GPT-2 small beam-search generate() call before and after fuse() (the "
                         "benchmark behind the reference's published numbers)")
    ap.add_argument("--fusion-dtype", default="fp32", choices=["fp32", "bf16"],
                    help="fusion: parameter dtype (the reference's script runs the fp32 checkpoint)")
    ap.add_argument("--prompt", type=int, default=512, help="decode: prompt length")
    ap.add_argument("--new-tokens", type=int, default=128, help="decode: tokens generated per call")
    ap.add_argument("--decode-batch", type=int, default=1, help="decode: sequences per call")
    ap.add_argument("--no-graph", action="store_true", help="decode: run the token loop eagerly (no CUDA graph)")
    ap.add_argument("--deployment", action="store_true",
                    help="decode: ONE ordinary process (no launcher); the model is created with deployment=True, which "
                         "spawns one worker per GPU, and generate() is called on the parent's handle")
    ap.add_argument("--hang-dump", type=float, default=0.0,
                    help="debugging: after this many seconds write every thread's Python stack to "
                         "<--hang-dump-dir>/hang_<HANG_TAG>_rank<r>.txt")
    ap.add_argument("--hang-dump-dir", default=".", help="where --hang-dump writes (default: the working directory)")
    ap.add_argument("--layers", type=int, default=None, help="profiling only: override the layer count (result is labelled debug)")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int) -> None:
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self) -> None:
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.2)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def reference_arm(args) -> None:
    """Run the unmodified reference through its own public API, or say why it cannot run here."""
    from baseline import reference_runner
    if args.mode == "train" and args.tp is None and args.pp is None:
        # the same sweep as this framework's arm: single, tp2, tp4, tp2 x pp4 (16 micro-batches of 4 sequences)
        spec, _ = default_plan(args.gpus)
        args.tp, args.pp = spec["tp"], spec["pp"]
        if spec.get("micro") and spec["pp"] > 1:
            args.micro_batch = args.micro_batch or spec["micro"]
    reference_runner.main(args, ClockSampler)


def default_plan(world: int):
    """Configurations timed by ``bench.py --gpus N`` with no parallelism flag: the GPT-J-6B sweep (one GPU, tensor
    parallel on 2 and 4, tensor x pipeline parallel on 8, 8 sequences of 2048 tokens per GPU per step) as the
    headline, and the other named 6B configurations of the same GPU count as extra blocks of the same line."""
    dp_block = dict(name=f"dp{world}_zero1", tp=1, pp=1)
    if world == 1:
        return dict(name="single", tp=1, pp=1), []
    if world == 2:
        return dict(name="tp2", tp=2, pp=1), [dp_block]
    if world == 4:
        return dict(name="tp4", tp=4, pp=1), [dp_block]
    if world == 8:
        # global batch 64 x 2048 as 16 micro-batches of 4 sequences through 4 stages of 7 layers, each stage on 2 GPUs
        # (extra blocks: the data-parallel one first, it is the same code as on 2 and 4 GPUs; last GPT-Neo 1.3B as
        # tp2 x pp2 x dp2 with 8 micro-batches of 4 sequences per replica and step)
        return (dict(name="tp2xpp4", tp=2, pp=4, micro=4),
                [dp_block, dict(name="tp8_b8x2048", tp=8, pp=1, replica_batch=8, micro=8),
                 dict(name="gptneo1.3b_tp2xpp2xdp2", model="gpt-neo-1.3b", tp=2, pp=2, replica_batch=32, micro=4)])
    return dp_block, []


def run_train_config(args, spec, dims, world, rank, local, dev):
    """Build GPT-J with the parallel layout ``spec``, time ``--steps`` steps twice (device inputs; end to end through
    pinned host memory), free everything again. Returns the result block (same keys on every rank)."""
    import gc

    import torch
    import torch.distributed as dist

    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel

    model_name = spec.get("model", args.model)
    if "model" in spec and spec["model"] != args.model:
        dims = MODELS[model_name]                       # an extra block on another architecture, always at full size
    n_layer, n_embd, n_head, rotary, vocab, n_pos = dims
    tp, pp = spec["tp"], spec["pp"]
    dp = world // (tp * pp)
    if model_name.startswith("gpt-neo"):
        cfg = ob.GPTNeoConfig(vocab_size=vocab, max_position_embeddings=n_pos, hidden_size=n_embd, num_layers=n_layer,
                              num_heads=n_head, window_size=256, attention_types=[[["global", "local"], n_layer // 2]],
                              torch_dtype=torch.bfloat16, use_cache=False)
        model_cls = ob.GPTNeoForCausalLM
    else:
        cfg = ob.GPTJConfig(vocab_size=vocab, n_positions=n_pos, n_embd=n_embd, n_layer=n_layer, n_head=n_head,
                            rotary_dim=rotary, torch_dtype=torch.bfloat16, use_cache=False)
        model_cls = ob.GPTJForCausalLM
    # sequences one model replica handles per step: weak scaling keeps 8 per GPU unless the configuration names a batch
    seqs_per_rank = spec.get("replica_batch") or args.batch_per_gpu * tp * pp
    # 4 sequences per forward/backward per GPU keeps activations within memory; tensor-parallel replicas spread a
    # micro-batch over tp GPUs, so they take proportionally more (fewer, larger launches)
    micro = spec.get("micro") or args.micro_batch or (4 * tp if model_name == "gptj-6b" else seqs_per_rank)
    micro = min(micro, seqs_per_rank)
    accum = seqs_per_rank // micro

    partition = None
    if pp > 1 and not args.even_partition:
        from oslo_b200.parallel.engine_pipeline import balanced_partition
        partition = balanced_partition(n_layer, pp)      # LM head + loss count as 1.5 blocks, the embedding as 0.15
    model = model_cls.from_config_with_parallel(
        cfg, tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=micro, seed=1234,
        init_on_device=True, torch_dtype=torch.bfloat16, pipeline_partition=partition)
    model.fuse()
    model.train()
    if args.checkpoint_activations:
        model.gradient_checkpointing_enable()
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0,
                     shard_group=mpu.get_data_parallel_group() if dp > 1 else None,
                     model_parallel_group=mpu.get_model_parallel_group() if tp * pp > 1 else None)
    engine = DistributedDataParallel(model, mpu, optimizer=opt) if dp > 1 else None
    call = engine if engine is not None else model

    gen = torch.Generator().manual_seed(1000 + mpu.get_data_parallel_rank())
    n_host = 4
    host = [torch.randint(0, vocab, (seqs_per_rank, args.seq), generator=gen).pin_memory() for _ in range(n_host)]
    dev_inputs = [h.to(dev) for h in host]
    ext = ob.ops.load_ext(required=True)

    def train_step(ids):
        opt.zero_grad()
        total = None
        if pp > 1:
            for out in call(input_ids=ids, labels=ids, output_logits=False):
                (out.loss / accum).backward()
                total = out.loss.detach() if total is None else total + out.loss.detach()
        else:
            for i in range(accum):
                mb = ids[i * micro:(i + 1) * micro]
                hold = engine.no_sync() if (engine is not None and i < accum - 1) else contextlib.nullcontext()
                with hold:  # gradients are reduced over the data-parallel group during the last backward only
                    loss = call(input_ids=mb, labels=mb, output_logits=False).loss
                    (loss / accum).backward()
                total = loss.detach() if total is None else total + loss.detach()
        opt.step()
        return total / accum

    def timed(steps, e2e):
        dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        sampler.start()
        l0 = ext.launch_count()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        t0.record()
        last = None
        for s in range(steps):
            if e2e:
                ids = host[s % n_host].to(dev, non_blocking=True)
                last = float(train_step(ids).item())
            else:
                last = train_step(dev_inputs[s % n_host])
        t1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        dist.barrier()
        clocks = sampler.stop()
        ms = torch.tensor([t0.elapsed_time(t1) if not e2e else wall * 1e3], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps, clocks, ext.launch_count() - l0, last

    for _ in range(args.warmup):
        train_step(dev_inputs[0])
    ms_step, clocks, launches, last = timed(args.steps, e2e=False)
    tokens_step = dp * seqs_per_rank * args.seq
    e2e = None
    if not args.no_e2e:
        ms_e2e, _, _, loss_host = timed(args.steps, e2e=True)
        e2e = {"value": tokens_step / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": seqs_per_rank * args.seq * 8, "d2h_bytes_per_step": 4, "last_loss": loss_host}
    pipe = None
    if pp > 1:
        # one more step with CUDA events around every forward / backward of every stage: how much of the step a stage
        # sits idle, against the 1F1B ideal (P - 1) / (m + P - 1)
        eng = model._pipe_engine
        eng.profile = True
        train_step(dev_inputs[0])
        torch.cuda.synchronize()
        rep = eng.schedule_report()
        eng.profile = False
        reps = [None] * world
        dist.all_gather_object(reps, rep)
        by_stage = {}
        for r in reps:
            by_stage.setdefault(r["stage"], []).append(r)
        pipe = {"stages": pp, "micro_batches": accum, "blocks_per_stage": partition or [n_layer // pp] * pp,
                "ideal_idle_share": round((pp - 1) / (accum + pp - 1), 4),
                "busy_ms_per_stage": [round(max(x["busy_ms"] for x in by_stage[s]), 1) for s in sorted(by_stage)],
                "idle_share_of_step": [round(1.0 - max(x["busy_ms"] for x in by_stage[s]) / ms_step, 4)
                                       for s in sorted(by_stage)]}
    err = torch.tensor([int(ext.error_word(dev_inputs[0]).item())], device=dev)
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], device=dev)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    par = "x".join(f"{k}{v}" for k, v in (("tp", tp), ("pp", pp), ("dp", dp)) if v > 1) or "single"
    from oslo_b200.config import get_config
    # model FLOPs of a step (6 x matrix parameters x tokens + the attention products, no recomputation counted) against
    # the measured GEMM throughput of this machine; never allowed to cost the measurement
    try:
        from oslo_b200.utils.metrics import load_measured_peaks, transformer_train_flops
        flops = transformer_train_flops(12.0 * n_layer * n_embd ** 2 + float(vocab) * n_embd, tokens_step, n_layer, n_embd,
                                        args.seq)
        peaks = load_measured_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
        per_gpu = flops / (ms_step / 1e3) / world / 1e12
        util = {"model_tflops_per_gpu": round(per_gpu, 1),
                "of_sustained_gemm_throughput": round(per_gpu / peaks["bf16_tflops_sustained"], 3),
                "peaks": peaks["source"]}
    except Exception as e:  # noqa: BLE001
        util = {"error": f"{type(e).__name__}: {e}"[:120]}
    block = {
        "value": tokens_step / (ms_step / 1e3), "unit": "tokens/s", "ms_per_step": ms_step,
        "config": {"model": model_name, "global_batch": dp * seqs_per_rank, "seq_len": args.seq,
                   "parallelism": par + ("+zero1" if dp > 1 else ""), "micro_batch": micro, "grad_accum": accum,
                   "optimizer": "AdamW fp32 master (fused)", "activation_checkpointing": bool(args.checkpoint_activations),
                   "fused_tp_collectives": bool(get_config().fused_tp_comm) if tp > 1 else None,
                   "pipeline": pipe, "utilisation": util,
                   "l2": "working set per step >> 126 MB L2, no explicit flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "device_error_word": int(err.item()),
        "peak_mem_gb": round(float(mem.item()), 1),
    }
    # free the model, the optimizer state and the symmetric workspaces before the next configuration is built
    del model, opt, engine, call, dev_inputs, host, train_step, timed
    from oslo_b200.parallel import fused_tp, symmetric
    fused_tp._CONTEXTS.clear()
    symmetric._WORKSPACES.clear()
    symmetric._CE_COMBINERS.clear()
    ext.set_reserved_sms(0)          # a pipeline-parallel configuration keeps a few SMs off the GEMM grids; the next one decides anew
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    dist.barrier()
    return block


def main() -> None:
    args = parse_args()
    if args.hang_dump > 0:
        import faulthandler
        os.makedirs(args.hang_dump_dir, exist_ok=True)
        f = open(os.path.join(args.hang_dump_dir, f"hang_{os.environ.get('HANG_TAG', 'x')}_rank{os.environ.get('RANK', '0')}.txt"), "w")
        faulthandler.dump_traceback_later(args.hang_dump, file=f, exit=False)
    if args.impl == "reference":
        reference_arm(args)
        return

    if args.mode == "decode" and args.deployment:
        decode_deployment_main(args)
        return
    if args.mode == "fusion":
        fusion_main(args)
        return

    import torch
    import torch.distributed as dist

    import oslo_b200 as ob  # noqa: F401
    from oslo_b200.parallel.mpu import MPU

    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run --nproc-per-node {args.gpus}")
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    n_layer, n_embd, n_head, rotary, vocab, n_pos = MODELS[args.model]
    if args.layers is not None:
        n_layer = args.layers
    dims = (n_layer, n_embd, n_head, rotary, vocab, n_pos)
    if args.mode == "decode":
        decode_main(args, world, rank, local, dev, dims)
        return
    if args.tp is None and args.pp is None:
        primary, extra = default_plan(world)
        if args.no_also:
            extra = []
    else:
        tp, pp = args.tp or 1, args.pp or 1
        primary, extra = dict(name="custom", tp=tp, pp=pp, replica_batch=args.replica_batch), []
    MPU.initialize_distributed("nccl")

    def emit(block, also):
        full = args.model == "gptj-6b" and args.layers is None
        name = {"gpt-neo-1.3b": "GPT-Neo-1.3B train tokens/sec"}.get(args.model if args.layers is None else "", f"{args.model} train tokens/sec (debug)")
        line = {
            "metric": "GPT-J-6B train tokens/sec" if full else name,
            "value": block["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": block["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights", "impl": "oslo_b200",
            "config": block["config"], "clocks": block["clocks"], "e2e": block["e2e"],
            "gpu_launches": block["gpu_launches"], "device_error_word": block["device_error_word"],
            "peak_mem_gb": block["peak_mem_gb"],
        }
        if also:
            line["also"] = also
        print(json.dumps(line), flush=True)

    t_primary = time.time()
    block = run_train_config(args, primary, dims, world, rank, local, dev)
    t_primary = time.time() - t_primary
    also = {}
    printed = threading.Event()

    def give_up():
        # an extra block that does not finish must not take the headline with it
        if printed.is_set():
            return
        printed.set()
        if rank == 0:
            emit(block, dict(also, error=f"extra configurations not finished within {also_limit:.0f} s"))
        sys.stdout.flush()
        os._exit(0)

    also_limit = max(args.also_timeout, 1.5 * t_primary * len(extra))
    guard = threading.Timer(also_limit, give_up) if extra else None
    if guard is not None:
        guard.daemon = True
        guard.start()
    for spec in extra:
        try:
            b = run_train_config(args, spec, dims, world, rank, local, dev)
            also[spec["name"]] = {k: b[k] for k in ("value", "unit", "ms_per_step", "e2e", "config", "gpu_launches",
                                                    "device_error_word", "peak_mem_gb")}
        except BaseException as e:  # noqa: BLE001 - the headline is measured already: an extra block must not lose it
            if isinstance(e, (KeyboardInterrupt, SystemExit)):
                raise
            also[spec["name"]] = {"error": f"{type(e).__name__}: {e}"[:300]}
            # after a failure in the middle of a step the ranks are no longer in step with one another (and a CUDA
            # error leaves no usable context): print what there is and leave without another collective. Ranks that
            # are still waiting for this one are released by their own timers.
            if guard is not None:
                guard.cancel()
            if rank == 0 and not printed.is_set():
                printed.set()
                emit(block, also)
            sys.stdout.flush()
            os._exit(0)
    if guard is not None:
        guard.cancel()
    if rank == 0 and not printed.is_set():
        printed.set()
        emit(block, also)
    dist.barrier()
    dist.destroy_process_group()


# seconds of one generate() call as printed in the reference's documentation and test docstrings; hardware not stated
# (USAGE.md:326-327, :339-340; tests/gpt2/gpt2_test_kernel_fusion.py:14-15, :62-63)
FUSION_PUBLISHED = {
    1: {"before_fuse_s": 3.5706350803375244, "after_fuse_s": 3.2512128353118896, "no_repeat_ngram_size": 4},
    4: {"before_fuse_s": 4.304628610610962, "after_fuse_s": 3.859266519546509,
        "after_fuse_fused_ngram_s": 3.620283210294232, "no_repeat_ngram_size": 2},
}


def fusion_main(args) -> None:
    """The reference's kernel-fusion benchmark (tests/gpt2/gpt2_test_kernel_fusion.py:11-107): GPT-2 small, one prompt,
    ``generate(max_length=200, min_length=200, num_beams=5, no_repeat_ngram_size=4)`` on one GPU, or tensor parallel
    over ``--gpus`` GPUs with ``no_repeat_ngram_size=2``, timed with the wall clock around the call (plus a device
    synchronize) before ``model.fuse()``, after it, and after it with ``fused_no_repeat_ngram_blocking=True``. Random
    weights instead of the hub checkpoint (``min_length`` pins the length, so the work per call is the same);
    ``--warmup`` full-length calls before each timing, mean over ``--steps`` calls, max over ranks. ``value`` is the
    after-fuse time; ``vs_baseline`` is it divided by the reference's published after-fuse time for the same GPU
    count (1 or 4; null otherwise)."""
    import torch
    import torch.distributed as dist

    import oslo_b200 as ob

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run --nproc-per-node {args.gpus}")
    on_gpu = torch.cuda.is_available() and os.environ.get("OSLO_B200_BACKEND", "nccl") != "gloo"
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if on_gpu:
        torch.cuda.set_device(local)
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[args.fusion_dtype]
    n_layer = args.layers if args.layers is not None else 12
    cfg = ob.GPT2Config(vocab_size=50257, n_positions=1024, n_embd=768, n_layer=n_layer, n_head=12, torch_dtype=dtype)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        model = ob.GPT2LMHeadModel.from_config_with_parallel(cfg, tensor_parallel_size=world, seed=1234,
                                                             init_on_device=on_gpu, torch_dtype=dtype)
        dev = model.mpu.device
    else:
        dev = torch.device("cuda", local) if on_gpu else torch.device("cpu")
        torch.manual_seed(1234)
        with torch.device(dev):
            model = ob.GPT2LMHeadModel._from_config(cfg, torch_dtype=dtype)
    model.eval()
    ngram = 4 if world == 1 else 2
    max_len = args.new_tokens + 8 if args.new_tokens != 128 else 200      # 200 as in the reference unless overridden
    prompt = torch.randint(0, 50257, (1, 8), generator=torch.Generator().manual_seed(7)).to(dev)
    kw = dict(max_length=max_len, min_length=max_len, num_beams=5, no_repeat_ngram_size=ngram, pad_token_id=0)

    def sync():
        if on_gpu:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def timed(**extra):
        for _ in range(5):
            model.generate(prompt, pad_token_id=0)                        # the reference's own warm-up: 5 default calls
        for _ in range(args.warmup):
            model.generate(prompt, **kw, **extra)
        sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            out = model.generate(prompt, **kw, **extra)
        sync()
        sec = (time.perf_counter() - t0) / args.steps
        if world > 1:
            t = torch.tensor([sec], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        assert out.shape == (1, max_len), out.shape
        return sec

    ext = ob.ops.load_ext(required=True) if on_gpu else None
    sampler = ClockSampler(local) if on_gpu else None
    if sampler is not None:
        sampler.start()
    before = timed()
    l0 = ext.launch_count() if ext is not None else 0
    model.fuse()
    after = timed()
    after_ngram = timed(fused_no_repeat_ngram_blocking=True)
    launches = (ext.launch_count() - l0) if ext is not None else 0
    clocks = sampler.stop() if sampler is not None else None
    pub = FUSION_PUBLISHED.get(world) if (n_layer == 12 and max_len == 200 and args.fusion_dtype == "fp32") else None
    if rank == 0:
        print(json.dumps({
            "metric": "GPT-2 small generate() seconds, 200 tokens, 5 beams, after fuse()" + ("" if n_layer == 12 and max_len == 200 else " (debug)"),
            "value": after, "unit": "s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": after * 1e3, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": (after / pub["after_fuse_s"]) if pub else None, "dtype": args.fusion_dtype,
            "data": "8 synthetic prompt token ids, random-init weights", "impl": "oslo_b200",
            "config": {"model": "gpt2-small", "parallelism": f"tp{world}" if world > 1 else "single", "num_beams": 5,
                       "max_length": max_len, "no_repeat_ngram_size": ngram, "batch": 1},
            "before_fuse_s": before, "after_fuse_s": after, "after_fuse_fused_ngram_s": after_ngram,
            "fuse_speedup": before / after, "published_reference": pub, "clocks": clocks, "gpu_launches": launches,
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def decode_deployment_main(args) -> None:
    """Greedy decoding through the deployment launcher, the way a serving script uses the package: this process is
    the only one the user starts; ``from_config_with_parallel(..., deployment=True)`` spawns one worker per GPU
    (tensor parallel over all of them) and ``model.generate(...)`` on the returned handle fans the request out.
    Timed in THIS process with the wall clock (request in, token ids out, through the worker queues). The per-token
    latency is the difference between a call that generates ``new_tokens`` tokens and one that generates a single
    token (prefill + first token), divided by ``new_tokens - 1``."""
    import torch

    import oslo_b200 as ob

    n_layer, n_embd, n_head, rotary, vocab, n_pos = MODELS[args.model]
    if args.layers is not None:
        n_layer = args.layers
    tp = args.tp or args.gpus
    cfg = ob.GPTJConfig(vocab_size=vocab, n_positions=n_pos, n_embd=n_embd, n_layer=n_layer, n_head=n_head,
                        rotary_dim=rotary, torch_dtype=torch.bfloat16, use_cache=True)
    model = ob.GPTJForCausalLM.from_config_with_parallel(cfg, tensor_parallel_size=tp, pipeline_parallel_size=1,
                                                         seed=1234, deployment=True, init_on_device=True,
                                                         torch_dtype=torch.bfloat16)
    model = model.fuse()
    b, prompt, n_new = args.decode_batch, args.prompt, args.new_tokens
    gen = torch.Generator().manual_seed(77)
    host = [torch.randint(0, vocab, (b, prompt), generator=gen) for _ in range(4)]
    try:
        def call(ids, new):
            return model.generate(ids, max_new_tokens=new, eos_token_id=None, pad_token_id=0,
                                  cuda_graph=not args.no_graph)

        def timed(steps, new):
            t0 = time.perf_counter()
            for s in range(steps):
                out = call(host[s % 4], new)
            return (time.perf_counter() - t0) * 1e3 / steps, out

        for _ in range(args.warmup):
            call(host[0], n_new)
            call(host[0], 1)
        ms_call, out = timed(args.steps, n_new)
        ms_first, _ = timed(args.steps, 1)
        assert tuple(out.shape) == (b, prompt + n_new), tuple(out.shape)
        ms_tok = (ms_call - ms_first) / max(n_new - 1, 1)
        full = args.model == "gptj-6b" and args.layers is None
        line = {
            "metric": f"GPT-J-6B TP={tp} decode ms/token" if full else f"{args.model} TP={tp} decode ms/token (debug)",
            "value": ms_tok, "unit": "ms/token", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_call, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights", "impl": "oslo_b200",
            "config": {"model": args.model, "global_batch": b, "seq_len": prompt, "new_tokens": n_new,
                       "parallelism": f"tp{tp}",
                       "decode": "deployment launcher: parent process -> worker queues -> generate(cuda_graph=" + str(not args.no_graph) + ")",
                       "timing": "wall clock in the parent process, host tensors in and out",
                       "prefill_plus_first_token_ms": ms_first, "tokens_per_s": b * 1e3 / ms_tok if ms_tok > 0 else None},
            "e2e": {"value": ms_call / n_new, "unit": "ms/token (whole generate call incl. prefill, host in/out)",
                    "ms_per_step": ms_call, "h2d_bytes_per_step": b * prompt * 8, "d2h_bytes_per_step": b * (prompt + n_new) * 8},
            "gpu_launches": None,
        }
        print(json.dumps(line), flush=True)
    finally:
        model.cpu()      # shuts the workers down


def decode_main(args, world, rank, local, dev, dims) -> None:
    """Greedy generation with a KV cache: tensor parallel over all GPUs, one CUDA-graph replay per token.

    A "step" is one ``generate`` call (prompt prefill + ``--new-tokens`` tokens). ``value`` is the decode latency
    per generated token after the prefill, device-timed, max over ranks; the end-to-end figure goes through
    pinned host memory for the prompt and copies the generated ids back to the host every call."""
    import torch
    import torch.distributed as dist

    import oslo_b200 as ob
    from oslo_b200.generation.graph_decode import GraphedGreedyDecoder

    n_layer, n_embd, n_head, rotary, vocab, n_pos = dims
    tp = args.tp or world
    cfg = ob.GPTJConfig(vocab_size=vocab, n_positions=n_pos, n_embd=n_embd, n_layer=n_layer, n_head=n_head,
                        rotary_dim=rotary, torch_dtype=torch.bfloat16, use_cache=True)
    model = ob.GPTJForCausalLM.from_config_with_parallel(cfg, tensor_parallel_size=tp, pipeline_parallel_size=1,
                                                         seed=1234, init_on_device=True, torch_dtype=torch.bfloat16)
    model.fuse()
    model.eval()
    ext = ob.ops.load_ext(required=True)
    b, prompt, n_new = args.decode_batch, args.prompt, args.new_tokens
    gen = torch.Generator().manual_seed(77)
    host = [torch.randint(0, vocab, (b, prompt), generator=gen).pin_memory() for _ in range(4)]
    dev_inputs = [h.to(dev) for h in host]
    dec = GraphedGreedyDecoder(model, max_len=prompt + n_new, use_graph=not args.no_graph)
    dec.record_events = True
    dec.launch_counter = ext.launch_count
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=rank, world_size=world)

    def timed(steps, e2e):
        dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        sampler.start()
        l0 = ext.launch_count()
        r0 = dec.replays
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        t0.record()
        decode_ms = prefill_ms = 0.0
        evs = []
        for s in range(steps):
            if e2e:
                ids = host[s % 4].to(dev, non_blocking=True)
                out = dec.generate(ids, n_new).cpu()
            else:
                out = dec.generate(dev_inputs[s % 4], n_new)
            evs.append(dec.events)
        t1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        for ev in evs:
            prefill_ms += ev[0].elapsed_time(ev[1])
            decode_ms += ev[1].elapsed_time(ev[2])
        dist.barrier()
        clocks = sampler.stop()
        tot = t0.elapsed_time(t1) if not e2e else wall * 1e3
        red = torch.tensor([tot, decode_ms, prefill_ms], device=dev)
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        tot, decode_ms, prefill_ms = red.tolist()
        launches = ext.launch_count() - l0 + (dec.replays - r0) * dec.kernels_per_step  # eager + replayed kernels
        return tot / steps, decode_ms / steps, prefill_ms / steps, clocks, launches, out

    for _ in range(args.warmup):
        dec.generate(dev_inputs[0], n_new)
    ms_call, ms_dec, ms_pre, clocks, launches, _ = timed(args.steps, e2e=False)
    e2e = None
    if not args.no_e2e:
        ms_e2e, _, _, _, _, out = timed(args.steps, e2e=True)
        e2e = {"value": ms_e2e / n_new, "unit": "ms/token (whole generate call incl. prefill, host in/out)",
               "ms_per_step": ms_e2e, "h2d_bytes_per_step": b * prompt * 8, "d2h_bytes_per_step": b * (prompt + n_new) * 8}
    err = int(ext.error_word(dev_inputs[0]).item())
    if rank == 0:
        full = args.model == "gptj-6b" and args.layers is None
        line = {
            "metric": f"GPT-J-6B TP={tp} decode ms/token" if full else f"{args.model} TP={tp} decode ms/token (debug)",
            "value": ms_dec / max(n_new - 1, 1), "unit": "ms/token", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_call, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "impl": "oslo_b200",
            "config": {"model": args.model, "global_batch": b, "seq_len": prompt, "new_tokens": n_new,
                       "parallelism": f"tp{tp}", "decode": "greedy, static KV cache, " + ("eager loop" if args.no_graph else "CUDA-graph step"),
                       "prefill_ms": ms_pre, "tokens_per_s": b * (n_new - 1) / (ms_dec / 1e3),
                       "l2": "weights + KV cache per token >> 126 MB L2 per GPU only at tp<=2; no explicit flush"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "device_error_word": err,
            "graph_replays": dec.replays, "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
        }
        print(json.dumps(line), flush=True)
    # captured graphs hold the tensor-parallel communicator: free them first, and do not let a slow communicator
    # shutdown keep a finished benchmark alive
    dec.release()
    import gc
    import threading
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    killer = threading.Timer(30.0, lambda: os._exit(0))
    killer.daemon = True
    killer.start()
    dist.destroy_process_group()
    killer.cancel()


if __name__ == "__main__":
    main()
