"""Per-step metrics (loss, tokens/s, TFLOP/s per GPU, memory) with a JSONL sink, and roofline helpers."""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

import torch


def load_measured_peaks(path: Optional[str] = None) -> Dict[str, float]:
    """Measured copy bandwidth / GEMM throughput of this machine when a ``MEASURED_PEAKS.json`` exists in the
    working directory, else the stated fallback (6.65 TB/s, 1.59 PFLOP/s burst, 1.4 sustained)."""
    path = path or os.path.join(os.getcwd(), "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def transformer_train_flops(n_params_dense: float, tokens: float, n_layer: int, n_embd: int, seq: int,
                            causal: bool = True) -> float:
    """6 * params * tokens for the dense GEMMs plus the attention score / value products (fwd + bwd)."""
    attn = 12.0 * n_layer * n_embd * seq * tokens * (0.5 if causal else 1.0)
    return 6.0 * n_params_dense * tokens + attn


def roofline_fraction(flops: float, nvlink_bytes: float, seconds: float, peak_tflops: float,
                      link_gbs: float = 770.0) -> Dict[str, float]:
    """Achieved fraction of the slower of (FLOPs / GEMM peak) and (NVLink bytes / link bandwidth)."""
    t_compute = flops / (peak_tflops * 1e12) if peak_tflops else 0.0
    t_link = nvlink_bytes / (link_gbs * 1e9) if link_gbs else 0.0
    bound = max(t_compute, t_link)
    return {"t_compute_s": t_compute, "t_link_s": t_link, "bound_s": bound,
            "fraction": bound / seconds if seconds > 0 else 0.0}


class MetricsLogger:
    def __init__(self, path: str = "", rank: Optional[int] = None) -> None:
        self.path = path
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self._t_last = time.perf_counter()

    def log_step(self, step: int, loss: Optional[float] = None, tokens: Optional[int] = None,
                 flops: Optional[float] = None, **extra: Any) -> Dict[str, Any]:
        now = time.perf_counter()
        dt = now - self._t_last
        self._t_last = now
        rec: Dict[str, Any] = {"step": step, "time_s": dt}
        if loss is not None:
            rec["loss"] = float(loss)
        if tokens is not None and dt > 0:
            rec["tokens_per_s"] = tokens / dt
        if flops is not None and dt > 0:
            rec["tflops_per_gpu"] = flops / dt / 1e12
        if torch.cuda.is_available():
            rec["mem_alloc_gb"] = torch.cuda.memory_allocated() / 2 ** 30
            rec["mem_peak_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
        rec.update(extra)
        if self.path and self.rank == 0:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec
