"""Micro-benchmark of the GEMM + collective kernels against GEMM followed by NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m oslo_b200.parallel.bench_fused_tp

Times every op with CUDA events on the launching stream (warm-up, a 256 MB write between iterations to
flush L2, max over ranks) on the per-rank shapes of a GPT-J layer at tensor-parallel size N, and prints one
JSON line per case with the achieved fraction of the roofline: the slower of FLOPs / measured GEMM peak and
NVLink bytes / 770 GB/s (measured peer-copy bandwidth per direction).
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist


def _time(fn, iters=10, warm=3):
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main() -> None:
    from oslo_b200.config import set_config
    from oslo_b200.ops import cuda_ops as co
    from oslo_b200.parallel.fused_tp import FusedTP
    from oslo_b200.parallel.mpu import MPU
    from oslo_b200.utils.metrics import load_measured_peaks

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    mpu = MPU(world, 1)
    g = mpu.get_tensor_parallel_group()
    peaks = load_measured_peaks()
    peak_tf, link = peaks["bf16_tflops"], 770.0
    M = int(os.environ.get("BENCH_TOKENS", 8192))
    H = 4096
    cases = [("row attn_out", M, H, H // world), ("row fc_out", M, H, 4 * H // world),
             ("col qkv+fc_in (merged)", M, 7 * H // world, H)]
    for use_mm in (True, False):
        set_config(use_multimem=use_mm)
        tp = FusedTP(g, workspace_mb=512)
        if use_mm and not tp.use_multimem:
            continue
        for name, m, n, k in cases:
            col = name.startswith("col")
            a = torch.randn(m // world if col else m, k, device="cuda").to(torch.bfloat16)
            b = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
            flops = 2.0 * m * n * k
            if col:
                full = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)

                def unfused():
                    dist.all_gather_into_tensor(full, a, group=g)
                    return co.gemm(full, b)

                def fused():
                    return tp.all_gather_gemm(a, b, False)[0]
                nv_bytes = (world - 1) / world * m * k * 2
                modes = [("all_gather->gemm", unfused, fused)]
            else:
                def unfused():
                    y = co.gemm(a, b)
                    dist.all_reduce(y, group=g)
                    return y

                def fused():
                    # the summed matrix is used where the kernel left it (a workspace slot), as the layers do
                    return tp.gemm_all_reduce(a, b, False, False, copy=False)

                def unfused_rs():
                    y = co.gemm(a, b)
                    out = torch.empty(m // world, n, device="cuda", dtype=torch.bfloat16)
                    dist.reduce_scatter_tensor(out, y, group=g)
                    return out

                def fused_rs():
                    return tp.gemm_reduce_scatter(a, b, False, False)
                nv_bytes = (world - 1) / world * m * n * 2
                modes = [("gemm->all_reduce", unfused, fused), ("gemm->reduce_scatter", unfused_rs, fused_rs)]
            t_gemm = _time(lambda: co.gemm(full if col else a, b))
            for op, fu, ff in modes:
                t_u, t_f = _time(fu), _time(ff)
                bound = max(flops / (peak_tf * 1e12), nv_bytes / (link * 1e9)) * 1e3
                if rank == 0:
                    print(json.dumps({"op": op, "layer": name, "tp": world, "multimem": tp.use_multimem, "M": m, "N": n,
                                      "K": k, "gemm_only_ms": round(t_gemm, 4), "gemm_then_nccl_ms": round(t_u, 4),
                                      "fused_ms": round(t_f, 4), "roofline_ms": round(bound, 4),
                                      "fused_frac_of_roofline": round(bound / t_f, 3),
                                      "peaks": peaks["source"]}), flush=True)
    err = int(torch.ops.oslo_b200.error_word(torch.zeros(1, device="cuda")).item())
    if rank == 0:
        print(json.dumps({"device_error_word": err}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    main()
