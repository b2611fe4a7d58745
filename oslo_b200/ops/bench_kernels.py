"""Micro-benchmarks of the hand-written kernels against library baselines, timed with CUDA events.

``python -m oslo_b200.ops.bench_kernels --op gemm``       tcgen05 GEMM vs ``torch.matmul`` (cuBLAS), GPT-J shapes
``python -m oslo_b200.ops.bench_kernels --op attention``  tcgen05 flash attention (forward, backward) vs the
                                                           mma.sync kernels of this package
``--case i`` restricts the run to one shape and ``--iters n --warmup w`` bound the number of launches, which is
what a profiler capture wants. Every line is JSON; ``frac_of_measured`` divides by the bf16 GEMM throughput in
``MEASURED_PEAKS.json`` at the repository root when that file exists (else by 1590 TFLOP/s).

Timing: ``warmup`` untimed calls, then ``iters`` calls each bracketed by events on the launching stream with a
write of a 256 MB buffer in between (L2 flush); the median is reported.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import cuda_ops as co
from . import load_ext

GEMM_CASES = [  # M, N, K, a_mn_major, b_mn_major
    (16384, 4096, 4096, 0, 0), (16384, 16384, 4096, 0, 0), (16384, 4096, 16384, 0, 0), (16384, 12288, 4096, 0, 0),
    (16384, 4096, 4096, 0, 1), (4096, 4096, 16384, 1, 1), (16384, 4096, 16384, 1, 1), (8192, 8192, 8192, 0, 0),
    (8192, 50400, 4096, 0, 0),
]
ATTN_CASES = [  # B, H, S, D
    (4, 16, 2048, 256), (4, 32, 2048, 128), (4, 32, 2048, 64), (1, 16, 8192, 256),
]


def _peak_tflops() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


class _Timer:
    def __init__(self, iters: int, warmup: int, flush: bool):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        ts = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]


def bench_gemm(args, timer: _Timer) -> None:
    peak = _peak_tflops()
    cases = GEMM_CASES if args.case is None else [GEMM_CASES[args.case]]
    for (M, N, K, amn, bmn) in cases:
        A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        a = A.t().contiguous() if amn else A
        b = B.t().contiguous() if bmn else B
        t = timer(lambda: co.gemm(a, b, bool(amn), bool(bmn)))
        rec = dict(op="gemm", M=M, N=N, K=K, a_mn_major=amn, b_mn_major=bmn, ms=round(t, 4),
                   tflops=round(2.0 * M * N * K / t / 1e9, 1))
        rec["frac_of_measured"] = round(rec["tflops"] / peak, 3)
        if not args.no_baseline:
            tb = timer(lambda: torch.matmul(a.t() if amn else a, b if bmn else b.t()))
            rec.update(cublas_ms=round(tb, 4), cublas_tflops=round(2.0 * M * N * K / tb / 1e9, 1))
        print(json.dumps(rec), flush=True)


def bench_attention(args, timer: _Timer) -> None:
    ext = load_ext(required=True)
    peak = _peak_tflops()
    cases = ATTN_CASES if args.case is None else [ATTN_CASES[args.case]]
    for (B, H, S, D) in cases:
        mk = lambda: (torch.randn(B, S, H, D, device="cuda") * 0.5).to(torch.bfloat16).permute(0, 2, 1, 3)
        q, k, v, do = mk(), mk(), mk(), mk()
        sc = 1.0 / math.sqrt(D)
        for causal in ((True, False) if args.causal is None else (bool(args.causal),)):
            o, lse = ext.flash_fwd(q, k, v, sc, causal, 0, None, 1)
            frac = 0.5 if causal else 1.0
            fl_f, fl_b = 4.0 * B * H * S * S * D * frac, 10.0 * B * H * S * S * D * frac
            tf = timer(lambda: ext.flash_fwd(q, k, v, sc, causal, 0, None, 1))
            tb = timer(lambda: ext.flash_bwd(do, q, k, v, o, lse, sc, causal, 0, None, 1))
            rec = dict(op="attention", B=B, H=H, S=S, D=D, causal=causal, fwd_ms=round(tf, 4), bwd_ms=round(tb, 4),
                       fwd_tflops=round(fl_f / tf / 1e9, 1), bwd_tflops=round(fl_b / tb / 1e9, 1))
            rec["fwd_frac_of_measured"] = round(rec["fwd_tflops"] / peak, 3)
            rec["bwd_frac_of_measured"] = round(rec["bwd_tflops"] / peak, 3)
            if not args.no_baseline:
                tf0 = timer(lambda: ext.flash_fwd(q, k, v, sc, causal, 0, None, 0))
                tb0 = timer(lambda: ext.flash_bwd(do, q, k, v, o, lse, sc, causal, 0, None, 0))
                rec.update(mma_sync_fwd_ms=round(tf0, 4), mma_sync_bwd_ms=round(tb0, 4))
            rec["device_error_word"] = int(ext.error_word(q).item())
            print(json.dumps(rec), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", choices=["gemm", "attention"], required=True)
    ap.add_argument("--case", type=int, default=None, help="index into the op's shape list")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--causal", type=int, default=None, help="attention: 1 / 0 to run only one mask")
    ap.add_argument("--no-baseline", action="store_true", help="skip the library / legacy-kernel baseline")
    ap.add_argument("--no-flush", action="store_true", help="do not write a 256 MB buffer between timed calls")
    args = ap.parse_args()
    timer = _Timer(args.iters, args.warmup, not args.no_flush)
    (bench_gemm if args.op == "gemm" else bench_attention)(args, timer)


if __name__ == "__main__":
    main()
