"""Merge a tensor- / pipeline-parallel checkpoint into one Hugging Face compatible ``pytorch_model.bin``.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/merge.py \
        --model gptj --checkpoint out --tp 2 --pp 2 --output out/merged --check

The directory ``--checkpoint`` holds the files ``save_pretrained_with_parallel`` wrote for that layout
(``pytorch_model_tp=i_pp=j.bin``). Every rank loads its own file, the de-parallel engines gather the shards, and
rank 0 writes the merged file. ``--check`` then loads the merged file into one unparallelized model on rank 0 and
compares its logits on a fixed random batch with the parallel model's.

It plays the role of the reference's ``tests/*/ *_test_tp_deparallelization.py`` / ``*_pp_*`` / ``*_3d_*`` scripts
(load a split checkpoint, generate, save merged, reload with ``tensor_parallel_size=1``, generate again), with a number
to look at instead of two texts. ``OSLO_B200_BACKEND=gloo`` runs it on CPU ranks.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import oslo_b200 as ob  # noqa: E402
from oslo_b200.utils import get_logger  # noqa: E402

CLASSES = {"gpt2": ob.GPT2LMHeadModel, "gpt_neo": ob.GPTNeoForCausalLM, "gptj": ob.GPTJForCausalLM}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="gptj", choices=sorted(CLASSES))
    ap.add_argument("--checkpoint", required=True, help="directory with the split files")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--pipeline-partition", default=None, help="blocks per stage the checkpoint was written with, e.g. 7,7,8,6")
    ap.add_argument("--output", required=True, help="directory for the merged checkpoint")
    ap.add_argument("--check", action="store_true", help="compare the merged model's logits with the parallel model's")
    args = ap.parse_args()
    log = get_logger()
    on_gpu = torch.cuda.is_available() and os.environ.get("OSLO_B200_BACKEND", "nccl") != "gloo"
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    par = dict(tensor_parallel_size=args.tp, pipeline_parallel_size=args.pp, micro_batch_size=2)
    if args.pipeline_partition:
        par["pipeline_partition"] = [int(n) for n in args.pipeline_partition.split(",")]
    model = CLASSES[args.model].from_pretrained_with_parallel(args.checkpoint, **par).eval()
    model.save_pretrained_with_parallel(args.output, save_with_merging=True)
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        log.info("merged checkpoint written to %s", args.output)
    if args.check:
        ids = torch.randint(0, model.config.vocab_size, (2, 16), generator=torch.Generator().manual_seed(0))
        with torch.no_grad():
            out = model(input_ids=ids.to(model.mpu.device))
            if args.pp > 1:
                out = [o for o in out][0]              # every stage returns the last stage's output
        logits = out.logits.float().cpu()
        if dist.is_initialized():
            dist.barrier()                              # the merged file is complete
        if rank == 0:
            single = CLASSES[args.model].from_pretrained(args.output).eval()
            with torch.no_grad():
                want = single(input_ids=ids).logits.float()
            diff = float((logits - want).abs().max())
            scale = float(want.abs().max())
            print(f"max |parallel - merged| logit difference: {diff:.3e} (largest logit {scale:.3e})")
            if diff > 2e-2 * max(scale, 1.0):
                raise SystemExit("the merged model does not reproduce the parallel model")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
