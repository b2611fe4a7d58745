"""3D-parallel training from a config or a checkpoint, with ZeRO-1, checkpoints and bit-exact resume.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/train.py \
        --model gptj --config config.json --tp 2 --pp 2 --micro-batch-size 2 --batch-size 8 --seq 2048 \
        --data corpus --steps 1000 --save out --save-every 200

``--save-every`` writes checkpoint generations ``out/checkpoints/step-XXXXXXXX`` with a pointer to the newest complete
one; ``--auto-resume`` continues from it when it exists, so that

    python -m torch.distributed.run --max-restarts 3 ... examples/train.py ... --save out --save-every 200 --auto-resume

restarts itself from its last checkpoint after a rank has died (torchrun re-launches all workers).

``--data`` is the prefix of a ``.bin`` / ``.idx`` pair written by ``examples/preprocess.py``; without it the
script trains on synthetic token ids. ``--tiny`` replaces the config by a few-layer model (used by the CPU
test of this script: ``OSLO_B200_BACKEND=gloo`` runs the same code on CPU ranks).

It plays the role of the reference's ``tests/*/ *_test_3d_training.py`` scripts (model from
``from_pretrained_with_parallel``, data-parallel wrapper around ``gpu_modules()``, the micro-batch loss
generator under pipeline parallelism), with this framework's own optimizer and data-parallel wrapper.
"""
from __future__ import annotations

import argparse
import contextlib
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import oslo_b200 as ob  # noqa: E402
from oslo_b200.optim import DynamicLossScaler, FusedAdamW  # noqa: E402
from oslo_b200.parallel.data_parallel import DistributedDataParallel  # noqa: E402
from oslo_b200.utils import CheckpointManager, MetricsLogger, get_logger  # noqa: E402

FAMILIES = {
    "gpt2": (ob.GPT2Config, ob.GPT2LMHeadModel, dict(n_embd=64, n_layer=4, n_head=4)),
    "gpt_neo": (ob.GPTNeoConfig, ob.GPTNeoForCausalLM,
                dict(hidden_size=64, num_layers=4, num_heads=4, attention_types=[[["global", "local"], 2]],
                     window_size=16, max_position_embeddings=128)),
    "gptj": (ob.GPTJConfig, ob.GPTJForCausalLM, dict(n_embd=64, n_layer=4, n_head=4, rotary_dim=8)),
}
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="gptj", choices=sorted(FAMILIES))
    ap.add_argument("--config", help="HF-style config.json of the model family")
    ap.add_argument("--init", help="checkpoint directory to start from (merged or split files)")
    ap.add_argument("--tiny", action="store_true", help="a 4-layer, 64-wide model with a 260-token vocabulary")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--pipeline-partition", default=None,
                    help="blocks per pipeline stage: 'balanced' (fewer blocks where the LM head and the loss run), a "
                         "comma-separated list such as 7,7,8,6, or nothing for the even split")
    ap.add_argument("--batch-size", type=int, default=8, help="sequences per model replica per step")
    ap.add_argument("--micro-batch-size", type=int, default=None)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--dtype", default=None, choices=sorted(DTYPES), help="default: bf16 on GPUs, fp32 on CPU")
    ap.add_argument("--checkpoint-activations", action="store_true")
    ap.add_argument("--data", help="prefix of a preprocessed corpus (.bin/.idx)")
    ap.add_argument("--save", help="directory for checkpoints")
    ap.add_argument("--save-every", type=int, default=0)
    ap.add_argument("--merge", action="store_true", help="also write one merged HF-compatible pytorch_model.bin")
    ap.add_argument("--resume", action="store_true",
                    help="continue from the newest complete periodic checkpoint under <--save>/checkpoints, or from the "
                         "final checkpoint in --save when there is none")
    ap.add_argument("--auto-resume", action="store_true",
                    help="continue from the newest complete periodic checkpoint under <--save>/checkpoints if there is "
                         "one, else start fresh: with `torchrun --max-restarts N` a job that lost a rank restarts "
                         "itself from its last checkpoint")
    ap.add_argument("--keep", type=int, default=2, help="periodic checkpoints to keep (--save-every)")
    ap.add_argument("--fail-at-step", type=int, default=0,
                    help="testing: the last rank raises at this step during the first launch attempt (host-side fault "
                         "injection for --auto-resume; restarts see TORCHELASTIC_RESTART_COUNT > 0 and run through)")
    ap.add_argument("--metrics", help="JSONL file for per-step metrics (rank 0)")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--watchdog", action="store_true",
                    help="heartbeat through the rendezvous store: a rank that stops beating ends the others' next step "
                         "with RankFailure instead of a hang; device-side wait time-outs are raised after every step")
    return ap.parse_args()


def build_model(args, dtype):
    cfg_cls, model_cls, tiny = FAMILIES[args.model]
    par = dict(tensor_parallel_size=args.tp, pipeline_parallel_size=args.pp,
               micro_batch_size=args.micro_batch_size or args.batch_size, seed=args.seed,
               sequence_parallel=args.sequence_parallel)
    source = args.resume_dir or args.init
    if args.pipeline_partition and args.pp > 1:
        if args.pipeline_partition == "balanced":
            from oslo_b200.parallel.engine_pipeline import balanced_partition
            if args.tiny:
                blocks = cfg_cls(**tiny).num_hidden_layers
            else:
                blocks = (cfg_cls.from_pretrained(source) if source else cfg_cls.from_json_file(args.config)).num_hidden_layers
            par["pipeline_partition"] = balanced_partition(blocks, args.pp)
        else:
            par["pipeline_partition"] = [int(n) for n in args.pipeline_partition.split(",")]
    if source:
        return model_cls.from_pretrained_with_parallel(source, torch_dtype=dtype, **par)
    if args.tiny:
        cfg = cfg_cls(vocab_size=260, **({"n_positions": 128} if args.model != "gpt_neo" else {}), **tiny)
    elif args.config:
        cfg = cfg_cls.from_json_file(args.config)
    else:
        raise SystemExit("one of --config, --init, --tiny or --resume is needed")
    return model_cls.from_config_with_parallel(cfg, torch_dtype=dtype, init_on_device=torch.cuda.is_available(), **par)


def batches(args, mpu, vocab, device):
    """Yield ``[batch_size, seq]`` token ids for this data-parallel rank, forever."""
    dp_rank, dp = mpu.get_data_parallel_rank(), mpu.get_data_parallel_world_size()
    if args.data:
        from torch.utils.data import DataLoader, DistributedSampler
        from oslo_b200.data import DatasetForCausalLM, InfiniteDataLoader
        ds = DatasetForCausalLM(args.data, max_seq_length=args.seq, split_type="train", seed=args.seed)
        sampler = DistributedSampler(ds, num_replicas=dp, rank=dp_rank, shuffle=True, seed=args.seed, drop_last=True)
        loader = InfiniteDataLoader(DataLoader(ds, batch_size=args.batch_size, sampler=sampler, drop_last=True,
                                               pin_memory=device.type == "cuda"))
        for item in loader:
            yield item["input_ids"][:, :args.seq].to(device, non_blocking=True)
    else:
        gen = torch.Generator().manual_seed(args.seed + 17 * dp_rank)
        while True:
            yield torch.randint(0, vocab, (args.batch_size, args.seq), generator=gen).to(device)


def main() -> None:
    args = parse_args()
    log = get_logger()
    on_gpu = torch.cuda.is_available() and os.environ.get("OSLO_B200_BACKEND", "nccl") != "gloo"
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dtype = DTYPES[args.dtype or ("bf16" if on_gpu else "fp32")]
    # periodic checkpoints are generations under <save>/checkpoints with a pointer to the newest complete one; the final
    # checkpoint goes to <save> itself
    manager = CheckpointManager(os.path.join(args.save, "checkpoints"), keep=args.keep) if args.save else None
    args.resume_dir = args.save if args.resume else None
    if (args.resume or args.auto_resume) and manager is not None:
        from oslo_b200.parallel.mpu import MPU
        MPU.initialize_distributed()                    # the ranks agree on the generation every one of them can read
        args.resume_dir = manager.latest_usable(args.tp, args.pp) or args.resume_dir
    model = build_model(args, dtype)
    if on_gpu:
        model.fuse()
    model.train()
    if args.checkpoint_activations:
        model.gradient_checkpointing_enable()
    mpu = model.mpu
    dp, mp = mpu.get_data_parallel_world_size(), args.tp * args.pp
    params = list(model.gpu_parameters())
    groups = [dict(params=[p for p in params if p.dim() >= 2], weight_decay=0.1),      # matrices decay,
              dict(params=[p for p in params if p.dim() < 2], weight_decay=0.0)]       # biases and LayerNorm do not
    opt = FusedAdamW(groups, lr=args.lr, betas=(0.9, 0.95), max_grad_norm=1.0,
                     shard_group=mpu.get_data_parallel_group() if dp > 1 else None,
                     model_parallel_group=mpu.get_model_parallel_group() if mp > 1 else None, model=model,
                     loss_scaler=DynamicLossScaler() if dtype == torch.float16 else None)
    engine = DistributedDataParallel(model, mpu, optimizer=opt) if dp > 1 else model
    step0 = 0
    if args.resume_dir:
        step0 = model.load_training_state(args.resume_dir, opt)["step"]
        log.info("resumed from %s at step %d", args.resume_dir, step0)
    micro = args.micro_batch_size or args.batch_size
    accum = args.batch_size // micro
    scale = (lambda l: opt.loss_scaler.scale(l)) if opt.loss_scaler is not None else (lambda l: l)
    metrics = MetricsLogger(args.metrics or "")
    data = batches(args, mpu, model.config.vocab_size, mpu.device)
    beat = None
    if args.watchdog and dist.is_initialized() and dist.get_world_size() > 1:
        from torch.distributed.distributed_c10d import _get_default_store
        from oslo_b200.utils import Heartbeat
        beat = Heartbeat(_get_default_store(), dist.get_rank(), dist.get_world_size()).start()
    for _ in range(step0):          # a resumed run continues with the batch the interrupted one would have seen
        next(data)

    def save(step):
        if not args.save:
            return
        model.save_pretrained_with_parallel(args.save)
        model.save_training_state(args.save, opt, step=step)
        if args.merge:
            model.save_pretrained_with_parallel(os.path.join(args.save, "merged"), save_with_merging=True)

    first_attempt = os.environ.get("TORCHELASTIC_RESTART_COUNT", "0") == "0"
    for step in range(step0 + 1, args.steps + 1):
        if args.fail_at_step == step and first_attempt and dist.is_initialized() \
                and dist.get_rank() == dist.get_world_size() - 1:
            raise RuntimeError(f"injected failure at step {step} (--fail-at-step)")
        if beat is not None:
            beat.check_peers()      # host-side: raises before this rank enters a collective nobody will join
        ids = next(data)
        opt.zero_grad()
        total = 0.0
        if args.pp > 1:             # the forward is a generator: one loss per micro-batch, 1F1B underneath
            for out in engine(input_ids=ids, labels=ids, output_logits=False):
                scale(out.loss / accum).backward()
                total += float(out.loss.detach()) / accum
        else:
            for i in range(accum):
                mb = ids[i * micro:(i + 1) * micro]
                last = i == accum - 1
                hold = engine.no_sync() if (dp > 1 and not last) else contextlib.nullcontext()
                with hold:
                    loss = engine(input_ids=mb, labels=mb, output_logits=False).loss
                    scale(loss / accum).backward()
                total += float(loss.detach()) / accum
        stepped = opt.step()
        if on_gpu and args.watchdog:
            from oslo_b200.utils import raise_if_device_error
            raise_if_device_error(ids)
        rec = metrics.log_step(step, loss=total, tokens=dp * args.batch_size * args.seq, skipped=not stepped)
        log.info("step %d loss %.4f %.0f tokens/s", step, total, rec.get("tokens_per_s", 0.0))
        if args.save_every and step % args.save_every == 0 and step < args.steps:
            manager.save(model, opt, step)              # collective; the pointer moves when every rank has written
    save(args.steps)
    if args.save_every and manager is not None:
        manager.save(model, opt, args.steps)            # the newest generation is never older than the final checkpoint
    if beat is not None:
        beat.stop()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
