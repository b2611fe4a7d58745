"""Autograd wrappers around the sm_100a kernels (``torch.ops.oslo_b200``).

Every function here assumes CUDA tensors; ``oslo_b200.ops.functional`` routes CPU tensors to the
PyTorch statements instead. GEMM operand layouts (see ``csrc/gemm_sm100.cu``): ``a_mn`` / ``b_mn`` say
that the operand is stored with the contraction dim as rows, which lets forward, dgrad and wgrad of
both weight layouts run without a transpose copy.
"""
from __future__ import annotations

import itertools
import os
from typing import Optional

import torch
from torch import Tensor

from . import load_ext
from ..config import get_config as _get_config
from . import reference as ref

FLAG_BIAS, FLAG_GELU, FLAG_SAVE_PREACT, FLAG_DGELU, FLAG_RESIDUAL, FLAG_OUT_FP32, FLAG_ACCUMULATE = 1, 2, 4, 8, 16, 32, 64
_GELU = ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh")
_16BIT = (torch.bfloat16, torch.float16)
_dropout_calls = itertools.count()


class _CheckedOps:
    """Debug wrapper around the operator namespace (``OSLO_B200_DEBUG_SYNC=1``): every operator call is followed by a
    device synchronisation and a read of the per-device error word, so a kernel whose bounded wait ran out - or an
    asynchronous CUDA error - is reported at the call that caused it, with the operator's name, instead of at some
    later synchronisation point. The reference has nothing comparable (its kernels never wait on each other)."""

    def __init__(self, ext) -> None:
        self._ext = ext

    def __getattr__(self, name):
        fn = getattr(self._ext, name)
        if name in ("error_word", "launch_count"):
            return fn

        def checked(*args, **kwargs):
            out = fn(*args, **kwargs)
            if torch.cuda.is_current_stream_capturing():
                return out
            torch.cuda.synchronize()
            like = next((a for a in args if isinstance(a, Tensor) and a.is_cuda), None)
            if like is not None:
                code = int(self._ext.error_word(like).item())
                if code:
                    self._ext.error_word(like).zero_()
                    raise RuntimeError(f"oslo_b200 kernel behind `{name}` gave up a bounded wait (device error code {code})")
            return out

        return checked


_CHECKED = None


def _ext():
    ext = load_ext(required=True)
    if _get_config().debug_sync:
        global _CHECKED
        if _CHECKED is None or _CHECKED._ext is not ext:
            _CHECKED = _CheckedOps(ext)
        return _CHECKED
    return ext


def device_error_code(like: Tensor) -> int:
    """Code left by a kernel whose bounded wait ran out (0 = none). Synchronises the device."""
    return int(_ext().error_word(like).item())


def reset_device_error(like: Tensor) -> None:
    _ext().error_word(like).zero_()


def _as_operand(t: Tensor) -> Tensor:
    """2-D tensor with contiguous last dim, 16-byte aligned rows."""
    if t.stride(-1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16 or t.stride(0) < t.size(1):
        t = t.contiguous()
    return t


def gemm_ok(*ts: Tensor) -> bool:
    return all(t.dtype in _16BIT and t.size(-1) % 8 == 0 and t.size(0) > 0 for t in ts)


def gemm(a: Tensor, b: Tensor, a_mn: bool = False, b_mn: bool = False, bias: Optional[Tensor] = None,
         aux: Optional[Tensor] = None, out: Optional[Tensor] = None, aux_out: Optional[Tensor] = None,
         flags: int = 0, alpha: float = 1.0) -> Tensor:
    return _ext().gemm(_as_operand(a), _as_operand(b), int(a_mn), int(b_mn), bias, aux, out, aux_out, flags, alpha)


def gemm_nn(d: Tensor, w: Tensor) -> Tensor:
    """``d [n, V] @ w [V, H] -> [n, H]``."""
    return gemm(d, w, False, True)


def gemm_tn(d: Tensor, x: Tensor, out_dtype=None) -> Tensor:
    """``d[n, V].T @ x[n, H] -> [V, H]`` (fp32 output when ``out_dtype`` is float32)."""
    return gemm(d, x, True, True, flags=FLAG_OUT_FP32 if out_dtype == torch.float32 else 0)


SMALL_M_ROWS = 64  # inference calls with at most this many rows use the split-K path
GEMV_ROWS = 4      # ... and with at most this many rows the CUDA-core weight-streaming kernel


def weight_grad(weight: Tensor, a: Tensor, b: Tensor) -> Optional[Tensor]:
    """``a^T b`` (both ``[rows, *]``) as the gradient of ``weight``.

    Parameters whose ``.grad`` is a persistent, zeroed-per-step view of a flat buffer (marked
    ``_oslo_accum_grad`` by ``optim.FlatBuffers``) get the product accumulated into that view by the GEMM
    epilogue and ``None`` is returned, which spares the separate gradient tensor and the add kernel of every
    micro-batch; ``_oslo_grad_hook`` (set by the data-parallel wrapper) stands in for the post-accumulate hook
    that autograd does not call in that case."""
    g = weight.grad
    if (g is not None and getattr(weight, "_oslo_accum_grad", False) and g.dtype == weight.dtype
            and g.shape == weight.shape and g.is_contiguous() and not torch.is_grad_enabled()):
        gemm(a, b, True, True, out=g, flags=FLAG_ACCUMULATE)
        hook = getattr(weight, "_oslo_grad_hook", None)
        if hook is not None:
            hook(weight)
        return None
    return gemm(a, b, True, True)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, reversed_, gelu, residual=None):
        k = x.size(-1)
        x2 = x.reshape(-1, k)
        need_grad = any(ctx.needs_input_grad[:3])  # grad mode is always off inside forward(); ask the ctx
        flags = (FLAG_BIAS if bias is not None else 0) | (FLAG_GELU if gelu else 0)
        n = weight.size(1) if reversed_ else weight.size(0)
        res2 = None
        if residual is not None:   # y = x W^T + b + residual in the GEMM epilogue (no activation in between)
            flags |= FLAG_RESIDUAL
            res2 = residual.reshape(-1, n)
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
        z = None
        if gelu and need_grad:
            flags |= FLAG_SAVE_PREACT
            z = torch.empty(x2.size(0), n, dtype=x.dtype, device=x.device)
        # the result is allocated in its final shape and the GEMM writes through a 2-D view of it: a view RETURNED by
        # a custom function could not be modified in place afterwards (the in-place rotary does that to q and k)
        y = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
        gemm(x2, weight, False, reversed_, bias=bias, aux=res2, out=y.view(-1, n), aux_out=z, flags=flags)
        ctx.save_for_backward(x2, weight, z)
        ctx.reversed, ctx.has_bias, ctx.in_shape = reversed_, bias is not None, x.shape
        ctx.has_residual = residual is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight, z = ctx.saved_tensors
        ext = _ext()
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if z is not None:
            dy2 = ext.bias_gelu_bwd(dy2, z, None)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, False, not ctx.reversed).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = weight_grad(weight, x2, dy2) if ctx.reversed else weight_grad(weight, dy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ext.colsum(dy2).to(ctx.bias_dtype)
        d_res = dy if (ctx.has_residual and ctx.needs_input_grad[5]) else None
        return dx, dw, db, None, None, d_res


class _FusedMLP(torch.autograd.Function):
    """``fc_out(gelu(fc_in(x)))`` for ``[out, in]`` weights. The backward multiplies by ``gelu'`` inside the epilogue
    of fc_out's input-gradient GEMM instead of running a separate pass over the ``[rows, 4 * hidden]`` activation
    gradient."""

    @staticmethod
    def forward(ctx, x, w_in, b_in, w_out, b_out, residual=None):
        k = x.size(-1)
        x2 = x.reshape(-1, k)
        need_grad = any(ctx.needs_input_grad)
        flags = FLAG_GELU | (FLAG_BIAS if b_in is not None else 0)
        z = None
        if need_grad:
            flags |= FLAG_SAVE_PREACT
            z = torch.empty(x2.size(0), w_in.size(0), dtype=x.dtype, device=x.device)
        h = gemm(x2, w_in, False, False, bias=b_in, aux_out=z, flags=flags)
        y = torch.empty(*x.shape[:-1], w_out.size(0), dtype=x.dtype, device=x.device)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, w_out.size(0))
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
        gemm(h, w_out, False, False, bias=b_out, aux=res2, out=y.view(-1, w_out.size(0)),
             flags=(FLAG_BIAS if b_out is not None else 0) | (FLAG_RESIDUAL if residual is not None else 0))
        ctx.save_for_backward(x2, w_in, w_out, z, h)
        ctx.has_b_in, ctx.has_b_out, ctx.in_shape = b_in is not None, b_out is not None, x.shape
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w_in, w_out, z, h = ctx.saved_tensors
        ext = _ext()
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw_in = db_in = dw_out = db_out = None
        dz = gemm(dy2, w_out, False, True, aux=z, flags=FLAG_DGELU)      # (dy W_out) * gelu'(z)
        if ctx.needs_input_grad[3]:
            dw_out = weight_grad(w_out, dy2, h)
        if ctx.has_b_out and ctx.needs_input_grad[4]:
            db_out = ext.colsum(dy2).to(dy.dtype)
        if ctx.needs_input_grad[0]:
            dx = gemm(dz, w_in, False, True).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw_in = weight_grad(w_in, dz, x2)
        if ctx.has_b_in and ctx.needs_input_grad[2]:
            db_in = ext.colsum(dz).to(dy.dtype)
        d_res = dy if (ctx.has_residual and ctx.needs_input_grad[5]) else None
        return dx, dw_in, db_in, dw_out, db_out, d_res


def fused_mlp_ok(x: Tensor, w_in: Tensor, w_out: Tensor) -> bool:
    return (x.is_cuda and x.dtype in _16BIT and w_in.dtype == x.dtype and w_out.dtype == x.dtype and x.numel() > 0
            and x.size(-1) % 8 == 0 and w_in.size(0) % 8 == 0 and w_out.size(0) % 8 == 0
            and x.numel() // x.size(-1) > SMALL_M_ROWS)


def fused_mlp(x: Tensor, w_in: Tensor, b_in: Optional[Tensor], w_out: Tensor, b_out: Optional[Tensor],
              residual: Optional[Tensor] = None) -> Tensor:
    """``fc_out(gelu(fc_in(x))) (+ residual)``; the residual is added in fc_out's GEMM epilogue."""
    return _FusedMLP.apply(x, w_in, b_in, w_out, b_out, residual)


class _QKVLinear(torch.autograd.Function):
    """Three bias-free ``[out, in]`` projections of the same input. Forward is three GEMMs; the point is the
    backward: the three input-gradient GEMMs accumulate into one tensor in their epilogues instead of leaving two
    ``[rows, hidden]`` additions to autograd."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv):
        k = x.size(-1)
        x2 = x.reshape(-1, k)
        outs = []
        for w in (wq, wk, wv):
            y = torch.empty(*x.shape[:-1], w.size(0), dtype=x.dtype, device=x.device)
            gemm(x2, w, False, False, out=y.view(-1, w.size(0)))
            outs.append(y)
        ctx.save_for_backward(x2, wq, wk, wv)
        ctx.in_shape = x.shape
        return tuple(outs)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        x2, wq, wk, wv = ctx.saved_tensors
        dx = None
        dws = [None, None, None]
        for i, (d, w) in enumerate(((dq, wq), (dk, wk), (dv, wv))):
            if d is None:
                continue
            d2 = d.reshape(-1, d.size(-1))
            if not d2.is_contiguous():
                d2 = d2.contiguous()
            if ctx.needs_input_grad[0]:
                if dx is None:
                    dx = gemm(d2, w, False, True)
                else:
                    gemm(d2, w, False, True, out=dx, flags=FLAG_ACCUMULATE)
            if ctx.needs_input_grad[1 + i]:
                dws[i] = weight_grad(w, d2, x2)
        return (dx.view(ctx.in_shape) if dx is not None else None, *dws)


def qkv_linear(x: Tensor, wq: Tensor, wk: Tensor, wv: Tensor):
    return _QKVLinear.apply(x, wq, wk, wv)


def qkv_linear_ok(x: Tensor, *ws: Tensor) -> bool:
    return (x.is_cuda and x.dtype in _16BIT and x.numel() > 0 and x.size(-1) % 8 == 0
            and x.numel() // x.size(-1) > SMALL_M_ROWS and all(w.dtype == x.dtype and w.size(0) % 8 == 0 for w in ws))


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor], reversed_: bool, activation: Optional[str],
           residual: Optional[Tensor] = None) -> Tensor:
    """``act(x W^T + b)``; ``residual`` (no activation) is added in the GEMM epilogue on the large-input path."""
    if residual is not None:
        n_ = weight.size(1) if reversed_ else weight.size(0)
        big = (activation is None and x.is_cuda and x.dtype in _16BIT and weight.dtype == x.dtype and residual.dtype == x.dtype
               and x.size(-1) % 8 == 0 and n_ % 8 == 0 and x.numel() // max(x.size(-1), 1) > SMALL_M_ROWS
               and (bias is None or bias.dtype == x.dtype))
        if big:
            return _Linear.apply(x, weight, bias, reversed_, False, residual)
        return linear(x, weight, bias, reversed_, activation) + residual
    if activation is not None and activation not in _GELU:
        raise ValueError(f"unsupported fused activation {activation!r}")
    n = weight.size(1) if reversed_ else weight.size(0)
    ok = (x.dtype in _16BIT and weight.dtype == x.dtype and x.size(-1) % 8 == 0 and n % 8 == 0 and x.numel() > 0
          and (bias is None or bias.dtype == x.dtype))
    if not ok:  # fp32 or ragged shapes: library GEMM, same semantics
        return ref.linear(x, weight, bias, reversed_, activation)
    rows = x.numel() // x.size(-1)
    if rows <= SMALL_M_ROWS and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)):
        # decode steps: weight-streaming split-K GEMM so that every SM pulls weights, not just N / 128 of them
        x2 = _as_operand(x.reshape(rows, x.size(-1)))
        gelu_from = 0 if activation is not None else -1
        if rows <= GEMV_ROWS and not reversed_ and n % 4 == 0:
            y = _ext().gemv_rows(x2, None, _as_operand(weight), bias, gelu_from)   # no tensor-core tile to pad
        else:
            y = _ext().gemm_small_m(x2, _as_operand(weight), int(reversed_), bias, gelu_from)
        return y.view(*x.shape[:-1], n)
    return _Linear.apply(x, weight, bias, reversed_, activation is not None, None)


def small_m_ok(x: Tensor, *weights: Tensor) -> bool:
    """Whether an inference call with input ``x`` takes the few-row (decode) GEMM path."""
    if torch.is_grad_enabled() and (x.requires_grad or any(w.requires_grad for w in weights)):
        return False
    rows = x.numel() // max(x.size(-1), 1)
    return (x.is_cuda and x.dtype in _16BIT and 0 < rows <= SMALL_M_ROWS and x.size(-1) % 8 == 0
            and all(w.dtype == x.dtype and w.size(0) % 8 == 0 for w in weights))


def packed_linear_small_m(x: Tensor, weight: Tensor, bias: Optional[Tensor], gelu_from: int) -> Tensor:
    """``x @ weight^T + bias`` for a few rows with tanh-GeLU on output columns ``>= gelu_from`` (-1: none);
    ``weight`` is the row-wise concatenation of several ``[out_i, in]`` layers that share the input."""
    rows = x.numel() // x.size(-1)
    x2 = _as_operand(x.reshape(rows, x.size(-1)))
    if rows <= GEMV_ROWS and weight.size(0) % 4 == 0:
        y = _ext().gemv_rows(x2, None, _as_operand(weight), bias, int(gelu_from))
    else:
        y = _ext().gemm_small_m(x2, _as_operand(weight), 0, bias, int(gelu_from))
    return y.view(*x.shape[:-1], weight.size(0))


def gemv_two_inputs(x1: Tensor, x2: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
                    residual: Optional[Tensor] = None) -> Tensor:
    """``[x1 | x2] @ weight^T (+ bias) (+ residual)`` for at most ``GEMV_ROWS`` rows without materialising the
    concatenation."""
    return _ext().gemv_rows(_as_operand(x1), _as_operand(x2), _as_operand(weight), bias, -1, residual)


def rotary_append(q: Tensor, k: Tensor, v: Tensor, k_cache: Tensor, v_cache: Tensor, lengths: Tensor,
                  write_index: Tensor, rotary_dim: int, base: float = 10000.0) -> Tensor:
    """Decode step: rotary on the new token's ``q``/``k`` (``[B, heads*D]`` row slices, position ``lengths[b]``),
    ``k``/``v`` written into the static caches at ``write_index[0]``; returns the rotated ``q`` as ``[B, heads, D]``."""
    return _ext().rotary_append(q, k, v, k_cache, v_cache, lengths, write_index, int(rotary_dim), float(base))


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        xc = x.contiguous()
        y, mean, rstd = _ext().layernorm_fwd(xc, w, b, eps)
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.has_bias = b is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = _ext().layernorm_bwd(dy.contiguous(), xc, w, mean, rstd)
        return dx, dw, (db if ctx.has_bias else None), None


def layer_norm(x: Tensor, w: Tensor, b: Optional[Tensor], eps: float) -> Tensor:
    vec = 4 if x.dtype == torch.float32 else 8
    cols = x.size(-1)
    if x.dtype != w.dtype or cols % vec or cols // vec > 1024 or x.numel() == 0:
        return ref.layer_norm(x, w, b, eps)
    return _LayerNorm.apply(x, w, b, eps)


class _BiasGelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        xc = x.contiguous()
        ctx.save_for_backward(xc, bias)
        return _ext().bias_gelu_fwd(xc, bias)

    @staticmethod
    def backward(ctx, dy):
        xc, bias = ctx.saved_tensors
        dx = _ext().bias_gelu_bwd(dy.contiguous(), xc, bias)
        db = None
        if bias is not None and ctx.needs_input_grad[1]:
            db = _ext().colsum(dx.view(-1, dx.size(-1))).to(bias.dtype)
        return dx, db


def bias_gelu(x: Tensor, bias: Optional[Tensor]) -> Tensor:
    vec = 4 if x.dtype == torch.float32 else 8
    if x.size(-1) % vec or (bias is not None and bias.dtype != x.dtype) or x.numel() == 0:
        return ref.bias_gelu(x, bias)
    return _BiasGelu.apply(x, bias)


class _BiasDropoutResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed):
        ctx.p, ctx.seed = p, seed
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        r = residual.contiguous() if residual is not None else None
        return _ext().bias_dropout_residual(x.contiguous(), bias, r, p, seed, 0)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        dx = _ext().bias_dropout_residual(dy, None, None, ctx.p, ctx.seed, 1) if ctx.p > 0 else dy
        db = _ext().colsum(dx.view(-1, dx.size(-1))).to(ctx.bias_dtype) if ctx.has_bias else None
        return dx, db, (dy if ctx.has_res else None), None, None


def bias_dropout_residual(x: Tensor, bias: Optional[Tensor], residual: Optional[Tensor], p: float, training: bool) -> Tensor:
    vec = 4 if x.dtype == torch.float32 else 8
    p = float(p) if training else 0.0
    if x.size(-1) % vec or x.numel() == 0 or (bias is not None and bias.dtype != x.dtype) or \
            (residual is not None and (residual.dtype != x.dtype or residual.shape != x.shape)):
        return ref.bias_dropout_residual(x, bias, residual, p, training)
    # the mask is a hash of (seed, element index): the seed follows torch's seed and a call counter so that
    # tensor-parallel ranks, which run the same call sequence under one seed, drop the same elements
    seed = (torch.initial_seed() * 1000003 + next(_dropout_calls)) & 0x7FFFFFFFFFFFFFFF
    return _BiasDropoutResidual.apply(x, bias, residual, p, seed)


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, rotary_dim, base):
        ctx.save_for_backward(positions)
        ctx.rd, ctx.base = rotary_dim, base
        return _ext().rotary(x.contiguous(), positions, rotary_dim, base, False)

    @staticmethod
    def backward(ctx, dy):
        (positions,) = ctx.saved_tensors
        return _ext().rotary(dy.contiguous(), positions, ctx.rd, ctx.base, True), None, None, None


class _RotaryInplace(torch.autograd.Function):
    """Rotation of the first ``rotary_dim`` dims of every head, in place: the other dims (3/4 of a GPT-J head) are
    neither read nor written. The input is the fresh output of a projection that nothing else needs, and the
    incoming gradient is the attention kernel's own output, so both directions may overwrite their argument.
    ``x`` is any contiguous tensor laid out ``[tokens, heads, head_dim]`` in memory."""

    @staticmethod
    def forward(ctx, x, positions, heads, head_dim, rotary_dim, base):
        ctx.save_for_backward(positions)
        ctx.cfg = (heads, head_dim, rotary_dim, base)
        ctx.mark_dirty(x)
        _ext().rotary_(x, positions, heads, head_dim, rotary_dim, base, False)
        return x

    @staticmethod
    def backward(ctx, dy):
        (positions,) = ctx.saved_tensors
        heads, head_dim, rotary_dim, base = ctx.cfg
        if not dy.is_contiguous():
            dy = dy.contiguous()
        return _ext().rotary_(dy, positions, heads, head_dim, rotary_dim, base, True), None, None, None, None, None


def rotary_interleaved(x: Tensor, positions: Tensor, rotary_dim: int, base: float) -> Tensor:
    if positions.dim() == 1:
        positions = positions.unsqueeze(0).expand(x.size(0), -1)
    positions = positions.to(torch.long).contiguous()
    heads, head_dim = x.size(-2), x.size(-1)
    ok = (x.dim() == 4 and x.is_contiguous() and head_dim % 8 == 0 and rotary_dim % 8 == 0 and x.data_ptr() % 16 == 0
          and not x.is_leaf and os.environ.get("OSLO_B200_ROTARY_INPLACE", "1") != "0")
    if ok:
        target = x
        if x._is_view():
            # work on the tensor the view was taken from (typically the projection's [B, S, heads * head_dim] output):
            # autograd refuses in-place changes of views that a custom function returned, and a plain function output
            # needs no view bookkeeping at all
            base_t = x._base
            if (base_t is not None and base_t.is_contiguous() and base_t.numel() == x.numel()
                    and base_t.data_ptr() == x.data_ptr() and not base_t._is_view() and not base_t.is_leaf):
                target = base_t
            elif x.requires_grad:
                ok = False
        if ok:
            out = _RotaryInplace.apply(target, positions, heads, head_dim, rotary_dim, base)
            return out if target is x else out.view(x.shape)
    return _Rotary.apply(x, positions, rotary_dim, base)


def flash_supported(q: Tensor, k: Tensor, v: Tensor) -> bool:
    if q.dtype not in _16BIT or q.size(-1) not in (64, 128, 256) or q.numel() == 0:
        return False
    return q.dtype == k.dtype == v.dtype


def _flash_impl() -> int:
    """1 = tcgen05/TMEM forward kernel (default), 0 = the mma.sync kernel (``OSLO_B200_ATTN=mma``)."""
    return 0 if os.environ.get("OSLO_B200_ATTN", "tcgen05") == "mma" else 1


def _attn_operand(t: Tensor) -> Tensor:
    if t.stride(-1) != 1 or any(s % 8 for s in t.stride()[:-1]) or t.data_ptr() % 16:
        t = t.contiguous()
    return t


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale, kpm):
        q, k, v = _attn_operand(q), _attn_operand(k), _attn_operand(v)
        o, lse = _ext().flash_fwd(q, k, v, scale, causal, window, kpm, _flash_impl())
        ctx.save_for_backward(q, k, v, o, lse, kpm)
        ctx.cfg = (scale, causal, window)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, kpm = ctx.saved_tensors
        scale, causal, window = ctx.cfg
        dq, dk, dv = _ext().flash_bwd(_attn_operand(do), q, k, v, o, lse, scale, causal, window, kpm, _flash_impl())
        return dq, dk, dv, None, None, None, None


def flash_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, window: Optional[int], scale: float,
                    key_padding_mask: Optional[Tensor]) -> Tensor:
    kpm = None
    if key_padding_mask is not None:
        kpm = (key_padding_mask != 0).to(torch.uint8).contiguous()
    return _Flash.apply(q, k, v, bool(causal), int(window or 0), float(scale), kpm)


def decode_attention(q: Tensor, k_cache: Tensor, v_cache: Tensor, lengths: Tensor, scale: float,
                     window: Optional[int]) -> Tensor:
    return _ext().decode_attn(q.contiguous(), k_cache, v_cache, lengths.to(torch.int32), float(scale), int(window or 0))


class _CausalSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        y = _ext().causal_softmax_fwd(x.contiguous(), scale)
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return _ext().softmax_bwd(y, dy.contiguous(), ctx.scale), None


def causal_softmax(x: Tensor, scale: float) -> Tensor:
    return _CausalSoftmax.apply(x, float(scale))


class _MaskedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale):
        y = _ext().masked_softmax_fwd(x.contiguous(), mask, scale)
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return _ext().softmax_bwd(y, dy.contiguous(), ctx.scale), None, None


def masked_softmax(x: Tensor, mask: Tensor, scale: float) -> Tensor:
    return _MaskedSoftmax.apply(x, mask.to(torch.uint8).contiguous(), float(scale))


def ce_stats(logits: Tensor, labels: Tensor, vocab_start: int):
    return _ext().ce_stats(logits, labels.contiguous(), int(vocab_start))


def ce_grad_(logits: Tensor, labels: Tensor, vocab_start: int, lse: Tensor, scale: Tensor) -> Tensor:
    return _ext().ce_grad_(logits, labels.contiguous(), int(vocab_start), lse.contiguous(), scale.contiguous())


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        lg = logits if logits.stride(-1) == 1 else logits.contiguous()
        mx, se, tg = ce_stats(lg, labels, 0)
        lse = torch.log(se) + mx
        valid = labels != ignore_index
        count = valid.sum().clamp(min=1).to(torch.float32)
        ctx.save_for_backward(lg, labels, lse, valid, count)
        return torch.where(valid, lse - tg, torch.zeros_like(lse)).sum() / count

    @staticmethod
    def backward(ctx, g):
        lg, labels, lse, valid, count = ctx.saved_tensors
        scale = (g.float() / count) * valid.to(torch.float32)
        return ce_grad_(lg.clone(), labels, 0, lse, scale), None, None


def cross_entropy(logits: Tensor, labels: Tensor, ignore_index: int) -> Tensor:
    if logits.dim() != 2 or logits.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return ref.cross_entropy(logits, labels, ignore_index)
    return _CrossEntropy.apply(logits, labels, ignore_index)


def linear_cross_entropy(hidden: Tensor, weight: Tensor, bias: Optional[Tensor], labels: Tensor, ignore_index: int,
                         chunk_rows: int) -> Tensor:
    from ..parallel.vocab_parallel import linear_cross_entropy as lce
    fused = hidden.dtype in _16BIT and weight.dtype == hidden.dtype and hidden.size(-1) % 8 == 0 \
        and weight.size(0) % 8 == 0
    return lce(hidden, weight, bias, labels, ignore_index, chunk_rows, fused=fused)


def ban_repeated_ngrams(tokens: Tensor, lprobs: Tensor, n: int) -> Tensor:
    if lprobs.dtype != torch.float32 or not lprobs.is_contiguous():
        return ref.ban_repeated_ngrams(tokens, lprobs, n)
    return _ext().ngram_ban_(tokens.to(torch.long).contiguous(), lprobs, int(n))
