"""Shape / dtype ("fake tensor") implementations of the ``torch.ops.oslo_b200`` operators.

The reference's binding module only checks shapes and dtypes at call time
(oslo/fused_kernels/bindings/pybind_kernels.cpp:26-177). The kernels here are registered for the CUDA dispatch key,
so registering fake implementations lets the operators be traced under ``FakeTensorMode`` / ``torch.export`` /
``torch.compile`` graph capture without touching a GPU: each function returns empty tensors with the shapes,
dtypes and strides the kernels produce.
"""
from __future__ import annotations

import torch

_DONE = False
_FLAG_OUT_FP32 = 32


def register() -> None:
    """Idempotent; called once after the extension has been loaded."""
    global _DONE
    if _DONE:
        return
    _DONE = True
    reg = torch.library.register_fake

    @reg("oslo_b200::gemm")
    def _(a, b, a_mn, b_mn, bias, aux, out, aux_out, flags, alpha):
        if out is not None:
            return out
        m = a.size(1) if a_mn else a.size(0)
        n = b.size(1) if b_mn else b.size(0)
        return a.new_empty((m, n), dtype=torch.float32 if (flags & _FLAG_OUT_FP32) else a.dtype)

    @reg("oslo_b200::gemm_small_m")
    def _(a, b, b_mn, bias, gelu_from):
        return a.new_empty((a.size(0), b.size(1) if b_mn else b.size(0)))

    @reg("oslo_b200::gemv_rows")
    def _(x1, x2, w, bias, gelu_from, res=None):
        return x1.new_empty((x1.size(0), w.size(0)))

    @reg("oslo_b200::layernorm_fwd")
    def _(x, w, b, eps):
        rows = x.numel() // max(x.size(-1), 1)
        stat = x.new_empty((rows,), dtype=torch.float32)
        return torch.empty_like(x), stat, torch.empty_like(stat)

    @reg("oslo_b200::layernorm_bwd")
    def _(dy, x, w, mean, rstd):
        return torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)

    @reg("oslo_b200::bias_gelu_fwd")
    def _(x, bias):
        return torch.empty_like(x)

    @reg("oslo_b200::bias_gelu_bwd")
    def _(dy, x, bias):
        return torch.empty_like(x)

    @reg("oslo_b200::colsum")
    def _(x):
        return x.new_empty((x.size(-1),), dtype=torch.float32)

    @reg("oslo_b200::rotary")
    def _(x, positions, rotary_dim, base, inverse):
        return torch.empty_like(x)

    @reg("oslo_b200::flash_fwd")
    def _(q, k, v, scale, causal, window, kpm, impl=1):
        b, h, sq, d = q.shape
        o = q.new_empty((b, sq, h, d)).permute(0, 2, 1, 3)     # [B, H, S, D] view of a [B, S, H, D] buffer
        return o, q.new_empty((b, h, sq), dtype=torch.float32)

    @reg("oslo_b200::flash_bwd")
    def _(dout, q, k, v, o, lse, scale, causal, window, kpm, impl=1):
        return (torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=q.device),
                torch.empty_strided(k.shape, k.stride(), dtype=k.dtype, device=k.device),
                torch.empty_strided(v.shape, v.stride(), dtype=v.dtype, device=v.device))

    @reg("oslo_b200::decode_attn")
    def _(q, kc, vc, lengths, scale, window):
        return torch.empty_like(q)

    @reg("oslo_b200::causal_softmax_fwd")
    def _(x, scale):
        return torch.empty_like(x)

    @reg("oslo_b200::masked_softmax_fwd")
    def _(x, mask, scale):
        return torch.empty_like(x)

    @reg("oslo_b200::softmax_bwd")
    def _(y, dy, scale):
        return torch.empty_like(y)

    @reg("oslo_b200::ce_stats")
    def _(logits, labels, vocab_start):
        s = logits.new_empty((logits.size(0),), dtype=torch.float32)
        return s, torch.empty_like(s), torch.empty_like(s)

    @reg("oslo_b200::sumsq")
    def _(x):
        return x.new_empty((1,), dtype=torch.float32)

    @reg("oslo_b200::gemm_ce_stats")
    def _(a, b, b_mn, bias, labels, vocab_start):
        s = a.new_empty((a.size(0),), dtype=torch.float32)
        return s, torch.empty_like(s), torch.empty_like(s)

    @reg("oslo_b200::gemm_ce_grad")
    def _(a, b, b_mn, bias, labels, vocab_start, lse, scale):
        return a.new_empty((a.size(0), b.size(1) if b_mn else b.size(0)))

    @reg("oslo_b200::error_word")
    def _(like):
        return like.new_empty((1,), dtype=torch.int32)

    @reg("oslo_b200::bias_dropout_residual")
    def _(x, bias, residual, p, seed, mode):
        return torch.empty_like(x)

    @reg("oslo_b200::rotary_")
    def _(x, positions, heads, head_dim, rotary_dim, base, inverse):
        return x

    @reg("oslo_b200::ce_grad_")
    def _(logits, labels, vocab_start, lse, scale):
        return logits

    @reg("oslo_b200::adam_step")
    def _(p, g, m, v, p_lp, lr, beta1, beta2, eps, wd, step, grad_scale, inv_scale):
        return None

    @reg("oslo_b200::ngram_ban_")
    def _(tokens, lprobs, n):
        return lprobs

    @reg("oslo_b200::rotary_append")
    def _(q, k, v, kc, vc, lengths, write_index, rotary_dim, base):
        return q.new_empty((kc.size(0), kc.size(1), kc.size(3)))

    @reg("oslo_b200::wait_probe")
    def _(flag, target, limit_ms):
        return flag.new_empty((1,), dtype=torch.int64)

    # collectives over symmetric memory: the data moves between GPUs inside the kernels; for tracing only the local
    # outputs matter (in-place operators return nothing)
    @reg("oslo_b200::gemm_comm")
    def _(a, b, a_mn, b_mn, bias, aux, aux_out, out, flags, alpha, M, N, K, peer_bufs_dev, own_buf, mc_base, data_off,
          flag_off, flag_bytes, rank, world, epoch, done_base, mode, use_multimem, trace):
        return 0

    @reg("oslo_b200::vocab_embed")
    def _(ids, weight, lo, hi, peer_ptrs_dev, mc_ptr, signal_ptrs_dev, counters, half_bytes, rank, world, use_multimem):
        return weight.new_empty((ids.numel(), weight.size(1)))

    @reg("oslo_b200::allreduce_oneshot")
    def _(x, peer_ptrs_dev, mc_ptr, signal_ptrs_dev, counters, stage_off, half_bytes, rank, world, use_multimem):
        return None

    @reg("oslo_b200::allreduce_symm")
    def _(peer_ptrs_dev, mc_ptr, signal_ptrs_dev, out, numel, rank, world, use_multimem):
        return None

    @reg("oslo_b200::ce_combine")
    def _(mx, se, tg, peer_ptrs_dev, signal_ptrs_dev, counters, cap, rank, world):
        return None

    @reg("oslo_b200::dp_reduce_scatter")
    def _(like, peer_ptrs_dev, mc_ptr, signal_ptrs_dev, lo, hi, shard, rank, world, use_multimem):
        return None

    @reg("oslo_b200::dp_all_gather")
    def _(like, peer_ptrs_dev, mc_ptr, signal_ptrs_dev, lo, hi, shard, rank, world, use_multimem):
        return None

