"""Generate text from a checkpoint: HF-style ``generate()`` (greedy, sampling, beam search) or the CUDA-graph
greedy decoder, optionally tensor-parallel or through the deployment launcher.

    python examples/generate.py --model gptj --checkpoint out/merged --prompt "Hello" --max-new-tokens 64
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/generate.py \
        --model gptj --checkpoint out --tp 4 --num-beams 5 --no-repeat-ngram-size 2
    python examples/generate.py --model gptj --checkpoint out/merged --tp 4 --deployment    # one parent, 4 GPU workers

Mirrors the reference's ``tests/*/ *_test_kernel_fusion.py`` / ``*_test_deployment.py`` usage. Prompts are encoded
as UTF-8 bytes unless ``--tokenizer`` names a Hugging Face tokenizer directory.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import oslo_b200 as ob  # noqa: E402

CLASSES = {"gpt2": ob.GPT2LMHeadModel, "gpt_neo": ob.GPTNeoForCausalLM, "gptj": ob.GPTJForCausalLM}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="gptj", choices=sorted(CLASSES))
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--deployment", action="store_true")
    ap.add_argument("--prompt", default="Hello")
    ap.add_argument("--tokenizer")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--num-beams", type=int, default=1)
    ap.add_argument("--do-sample", action="store_true")
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--no-repeat-ngram-size", type=int, default=None)
    ap.add_argument("--cuda-graph", action="store_true", help="greedy decoding as one CUDA-graph replay per token")
    args = ap.parse_args()

    if args.tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(args.tokenizer)
        encode, decode = (lambda s: tok.encode(s)), (lambda ids: tok.decode(ids))
    else:
        encode = lambda s: list(s.encode("utf-8"))                                            # noqa: E731
        decode = lambda ids: bytes(int(i) for i in ids if 0 <= int(i) < 256).decode("utf-8", "replace")  # noqa: E731

    on_gpu = torch.cuda.is_available() and os.environ.get("OSLO_B200_BACKEND", "nccl") != "gloo"
    cls = CLASSES[args.model]
    if args.tp > 1 or args.deployment:
        model = cls.from_pretrained_with_parallel(args.checkpoint, tensor_parallel_size=args.tp,
                                                  deployment=args.deployment or None)
        device = torch.device("cpu") if args.deployment else model.mpu.device
    else:
        model = cls.from_pretrained(args.checkpoint)
        device = torch.device("cuda") if on_gpu else torch.device("cpu")
        model = model.to(device)
    if on_gpu and not args.deployment:
        model.fuse()
    model.eval()
    ids = torch.tensor([encode(args.prompt)], dtype=torch.long, device=device)
    kw = dict(max_new_tokens=args.max_new_tokens, num_beams=args.num_beams, do_sample=args.do_sample,
              top_k=args.top_k, top_p=args.top_p, temperature=args.temperature,
              no_repeat_ngram_size=args.no_repeat_ngram_size)
    if args.cuda_graph:
        kw["cuda_graph"] = True
    if on_gpu and args.no_repeat_ngram_size:
        kw["fused_no_repeat_ngram_blocking"] = True
    t0 = time.perf_counter()
    out = model.generate(ids, **{k: v for k, v in kw.items() if v is not None})
    dt = time.perf_counter() - t0
    if int(os.environ.get("RANK", "0")) == 0:
        new = out[0, ids.size(1):].tolist()
        print(decode(out[0].tolist()))
        print(f"[{len(new)} new tokens in {dt:.2f} s]", file=sys.stderr)


if __name__ == "__main__":
    main()
