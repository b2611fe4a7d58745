"""LM-head projection fused with softmax cross-entropy, optionally over a vocabulary-sharded head.

The ``[tokens, vocab]`` logits are produced ``chunk_rows`` rows at a time and reduced to three
numbers per row (max, sum of exponentials, target logit). With a sharded vocabulary those are
combined over the tensor-parallel group (MAX / SUM / SUM all-reduces of ``[rows]`` vectors), so no
rank ever holds or gathers full logits - the reference all-gathers ``[B, S, V]`` instead
(oslo/parallelism/mpu.py:759, oslo/models/gpt2/modeling_gpt2.py:983-1019). The backward recomputes
each chunk of logits, forms ``softmax - onehot`` in place and feeds the two gradient GEMMs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .mpu import ceil_split_sizes


def _proj(x: Tensor, w: Tensor, b: Optional[Tensor], fused: bool) -> Tensor:
    if fused and x.is_cuda:
        from .. import ops
        return ops.linear(x, w, b)
    y = x @ w.t()
    return y if b is None else y + b


def _stats(logits: Tensor, labels: Tensor, lo: int, fused: bool):
    """Row max, sum(exp(l - max)) and the target logit (0 when the target is not in this shard)."""
    if fused and logits.is_cuda:
        from ..ops import cuda_ops
        return cuda_ops.ce_stats(logits, labels, lo)
    lf = logits.float()
    mx = lf.max(dim=-1).values
    se = torch.exp(lf - mx[:, None]).sum(-1)
    local = labels - lo
    inside = (local >= 0) & (local < logits.size(-1))
    tgt = lf.gather(1, local.clamp(0, logits.size(-1) - 1)[:, None]).squeeze(1)
    return mx, se, torch.where(inside, tgt, torch.zeros_like(tgt))


def _grad_inplace(logits: Tensor, labels: Tensor, lo: int, lse: Tensor, scale: Tensor, fused: bool) -> Tensor:
    """``(softmax - onehot) * scale`` written over ``logits`` (rows with ignored labels get zero)."""
    if fused and logits.is_cuda:
        from ..ops import cuda_ops
        return cuda_ops.ce_grad_(logits, labels, lo, lse, scale)
    p = torch.exp(logits.float() - lse[:, None])
    local = labels - lo
    inside = (local >= 0) & (local < logits.size(-1))
    rows = torch.nonzero(inside, as_tuple=True)[0]
    p[rows, local[rows]] -= 1.0
    p *= scale[:, None]
    logits.copy_(p)
    return logits


def shard_rows_aligned(full_vocab: int, tp: int) -> bool:
    """Every rank's vocabulary shard has a multiple of 8 rows (50400 over 2 or 4 ranks: yes; 50257 over 2: 25129 and
    25128, no; 50400 over 8: 6300, no). The same answer on every rank of the group."""
    return all(s % 8 == 0 for s in ceil_split_sizes(int(full_vocab), max(int(tp), 1)))


def _epilogue_ce_ok(hidden: Tensor, weight: Tensor, bias: Optional[Tensor], fused: bool, full_vocab: int, tp: int) -> bool:
    """The LM-head GEMM can do the cross-entropy work in its epilogue: kernels in use, 16-bit operands of one dtype,
    ``[vocab, hidden]`` weight with 16-byte aligned rows. The answer also selects the collective that combines the
    shards' statistics, so it must not depend on anything that differs between the ranks of the tensor-parallel group:
    the row count is checked for ALL shards, not for this rank's."""
    if not (fused and hidden.is_cuda and hidden.dtype in (torch.bfloat16, torch.float16)):
        return False
    if not shard_rows_aligned(full_vocab, tp):
        return False
    from ..config import get_config
    if not get_config().ce_in_gemm_epilogue:
        return False
    ok = (weight.dtype == hidden.dtype and weight.dim() == 2 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0
          and hidden.size(-1) % 8 == 0 and weight.data_ptr() % 16 == 0
          and weight.size(0) % 8 == 0)      # rows of the [rows, vocab shard] gradient matrix stay 16-byte aligned
    # (data_ptr alignment and strides of a shard come from the same allocator and the same slicing code on every rank)
    return ok and (bias is None or (bias.dtype == hidden.dtype and bias.is_contiguous()))


def _own_collectives() -> bool:
    from ..config import get_config
    return bool(get_config().fused_tp_comm)


def _one_node(mpu) -> bool:
    from .symmetric import group_on_one_node
    return group_on_one_node(mpu.get_tensor_parallel_group())


def _as_rows(x: Tensor) -> Tensor:
    return x if (x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0) else x.contiguous()


class _LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, bias, labels, mpu, full_vocab, ignore_index, chunk_rows, fused):
        tp = mpu.tp if mpu is not None else 1
        lo = 0
        if tp > 1:
            sizes = ceil_split_sizes(full_vocab, tp)
            lo = sum(sizes[: mpu.tp_rank])
        n = hidden.size(0)
        mx = torch.empty(n, dtype=torch.float32, device=hidden.device)
        se = torch.empty_like(mx)
        tg = torch.empty_like(mx)
        in_epilogue = _epilogue_ce_ok(hidden, weight, bias, fused, full_vocab, tp)
        for s in range(0, n, chunk_rows):
            e = min(n, s + chunk_rows)
            if in_epilogue:
                # per-row (max, sum exp, label logit) straight out of the GEMM's accumulators: no logits tensor
                from .. import ops
                mx[s:e], se[s:e], tg[s:e] = ops.load_ext(required=True).gemm_ce_stats(
                    _as_rows(hidden[s:e]), weight, 0, bias, labels[s:e].contiguous(), lo)
                continue
            lg = _proj(hidden[s:e], weight, bias, fused)
            mx[s:e], se[s:e], tg[s:e] = _stats(lg, labels[s:e], lo, fused)
        if tp > 1 and in_epilogue and mpu.backend == "nccl" and _own_collectives() and _one_node(mpu):
            # one kernel, one cross-rank meeting: peers' statistics read from symmetric memory and combined in place
            from .symmetric import get_ce_combine
            get_ce_combine(mpu.get_tensor_parallel_group(), hidden.device)(mx, se, tg)
        elif tp > 1:
            gmx = mx.clone()
            dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=mpu.get_tensor_parallel_group())
            se = se * torch.exp(mx - gmx)
            packed = torch.stack((se, tg))
            dist.all_reduce(packed, group=mpu.get_tensor_parallel_group())
            se, tg, mx = packed[0], packed[1], gmx
        lse = torch.log(se) + mx
        valid = labels != ignore_index
        count = valid.sum().clamp(min=1).to(torch.float32)
        loss = torch.where(valid, lse - tg, torch.zeros_like(lse)).sum() / count
        ctx.save_for_backward(hidden, weight, bias, labels, lse, valid, count)
        ctx.mpu, ctx.lo, ctx.chunk, ctx.fused = mpu, lo, chunk_rows, fused
        ctx.in_epilogue = in_epilogue
        return loss

    @staticmethod
    def backward(ctx, g):
        hidden, weight, bias, labels, lse, valid, count = ctx.saved_tensors
        mpu, lo, fused = ctx.mpu, ctx.lo, ctx.fused
        n = hidden.size(0)
        scale = (g.float() / count) * valid.to(torch.float32)
        dx = torch.empty_like(hidden)
        # the gradient GEMMs take [rows, vocab shard] operands: with a shard whose row count is not a multiple of 8 the
        # rows of that matrix are not 16-byte aligned and the library products below are used instead (a local choice)
        on_kernels = fused and hidden.is_cuda and weight.size(0) % 8 == 0
        dw = None if on_kernels else torch.zeros_like(weight, dtype=torch.float32)
        dw_acc = None
        # weights whose gradient lives in the optimizer's flat buffer take the chunks' products there directly
        direct_dw = (on_kernels and getattr(weight, "_oslo_accum_grad", False) and weight.grad is not None
                     and weight.grad.dtype == weight.dtype and weight.grad.is_contiguous() and ctx.needs_input_grad[1])
        db = torch.zeros(weight.size(0), dtype=torch.float32, device=weight.device) if bias is not None else None
        for s in range(0, n, ctx.chunk):
            e = min(n, s + ctx.chunk)
            x = hidden[s:e]
            if ctx.in_epilogue:
                # recomputed logits leave the GEMM as (softmax - onehot) * scale
                from .. import ops
                x = _as_rows(x)
                d = ops.load_ext(required=True).gemm_ce_grad(x, weight, 0, bias, labels[s:e].contiguous(), lo,
                                                            lse[s:e].contiguous(), scale[s:e].contiguous())
            else:
                lg = _proj(x, weight, bias, fused)
                d = _grad_inplace(lg, labels[s:e], lo, lse[s:e], scale[s:e], fused)
            if on_kernels:
                from ..ops import cuda_ops
                cuda_ops.gemm(d, weight, False, True, out=dx[s:e])      # written in place, no chunk copy
                if direct_dw:
                    # adds into the flat gradient buffer; only the last chunk goes through weight_grad, whose
                    # gradient-ready hook must fire once per backward pass
                    if e == n:
                        part = cuda_ops.weight_grad(weight, d, x)
                        if part is not None:   # the in-place route declined after all: add the product by hand
                            weight.grad.add_(part)
                    else:
                        cuda_ops.gemm(d, x, True, True, out=weight.grad, flags=cuda_ops.FLAG_ACCUMULATE)
                elif dw_acc is None:
                    dw_acc = cuda_ops.gemm_tn(d, x, out_dtype=torch.float32)
                else:                                                   # later chunks accumulate in the epilogue
                    cuda_ops.gemm(d, x, True, True, out=dw_acc, flags=cuda_ops.FLAG_OUT_FP32 | cuda_ops.FLAG_ACCUMULATE)
                if db is not None:
                    db += cuda_ops._ext().colsum(d)                     # fp32 column sums without an fp32 copy of d
            else:
                dx[s:e] = (d @ weight).to(dx.dtype)
                dw += d.float().t() @ x.float()
                if db is not None:
                    db += d.float().sum(0)
        if dw_acc is not None:
            dw = dw_acc
        if mpu is not None and mpu.tp > 1:
            dist.all_reduce(dx, group=mpu.get_tensor_parallel_group())
        return (dx, dw.to(weight.dtype) if dw is not None else None, db.to(bias.dtype) if db is not None else None,
                None, None, None, None, None, None)


def linear_cross_entropy(hidden: Tensor, weight: Tensor, bias: Optional[Tensor], labels: Tensor,
                         ignore_index: int = -100, chunk_rows: int = 4096, fused: bool = True) -> Tensor:
    return _LinearCrossEntropy.apply(hidden, weight, bias, labels, None, weight.size(0), ignore_index,
                                     chunk_rows, fused)


def vocab_parallel_linear_cross_entropy(hidden: Tensor, weight: Tensor, bias: Optional[Tensor], labels: Tensor,
                                        mpu, full_vocab: int, ignore_index: int = -100, chunk_rows: int = 4096,
                                        fused: bool = False) -> Tensor:
    """Mean loss over rows with a label; ``weight`` / ``bias`` hold this rank's vocabulary rows."""
    return _LinearCrossEntropy.apply(hidden, weight, bias, labels, mpu, full_vocab, ignore_index, chunk_rows, fused)
