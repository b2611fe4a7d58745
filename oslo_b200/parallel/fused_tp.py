"""Tensor-parallel linear layers whose collective runs INSIDE the GEMM kernel.

``FusedTP`` owns the symmetric workspace of one tensor-parallel group and exposes the three fused ops of
``csrc/fused_comm_gemm.cu``:

* ``gemm_all_reduce``      - row-parallel forward and column-parallel input-gradient (``sum_r x_r W_r``)
* ``gemm_reduce_scatter``  - the sequence-parallel form of the same product (each rank keeps its rows)
* ``all_gather_gemm``      - sequence-parallel column-parallel forward (``[x_0; x_1; ...] W``)

The autograd functions below use them for forward and backward, so one fused kernel replaces every
``matmul`` + NCCL all-reduce / all-gather pair of the reference's parallel layers
(oslo/modeling_utils.py:67-104, oslo/parallelism/mpu.py:848-890). ``N_SLOTS`` workspace slots are used in turn
(see the kernel's notes on why that makes reuse safe without a trailing barrier). The all-reduced matrix is handed
out as a VIEW of its slot, not as a copy: it stays valid until ``N_SLOTS - 1`` further fused calls have been issued
on this rank (a peer can only write into a slot again after this rank has itself reached the call before the one
that reuses it), which covers "consume it with the next elementwise op"; anything that must live longer - a
tensor saved for backward - has to be cloned by the caller.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from .. import ops
from ..config import get_config
from .symmetric import SymmetricWorkspace, group_on_one_node

MODE_ALLREDUCE, MODE_REDUCE_SCATTER, MODE_ALLGATHER = 1, 2, 3
_FLAG_RESIDUAL = 16            # GEMM epilogue flag: add the aux operand (here: another per-rank partial sum)
_FLAG_BYTES = 4 << 20          # readiness words (one per tile, rank and warp) + the completion counter, per slot
N_SLOTS = 4                    # workspace slots used in turn
_CONTEXTS: Dict[str, "FusedTP"] = {}


class FusedTP:
    def __init__(self, group, workspace_mb: Optional[int] = None) -> None:
        mb = workspace_mb or get_config().symm_buffer_mb
        self.group = group
        self.ws = SymmetricWorkspace(group, N_SLOTS * (mb * 2 ** 20 + _FLAG_BYTES))
        self.world, self.rank = self.ws.world, self.ws.rank
        self.slot_bytes = mb * 2 ** 20
        self.epochs = [0] * N_SLOTS
        self.done_totals = [0] * N_SLOTS
        self.calls = 0
        self.own_base = self.ws.buf.data_ptr()
        self.use_multimem = get_config().use_multimem and self.ws.has_multicast
        # set to an int64 [>= grid, 8] CUDA tensor to receive per-CTA phase timestamps (ns) of the next calls:
        # 0 start, 2 last MMA issued, 3 epilogue done, 4 communication done, 5 epilogue fence time,
        # 6 time the communication warps waited for tiles, 7 time they moved data
        self.trace: Optional[Tensor] = None

    def _next_slot(self) -> Tuple[int, int, int, int]:
        slot = self.calls % N_SLOTS
        self.calls += 1
        self.epochs[slot] += 1
        data_off = slot * (self.slot_bytes + _FLAG_BYTES)
        return slot, data_off, data_off + self.slot_bytes, self.epochs[slot]

    def fits(self, rows: int, cols: int) -> bool:
        return rows * cols * 2 <= self.slot_bytes and rows * cols > 0

    def _call(self, a, b, a_mn, b_mn, bias, aux_out, out, flags, M, N, K, mode, aux=None):
        slot, data_off, flag_off, epoch = self._next_slot()
        inc = ops.load_ext(required=True).gemm_comm(
            a, b, int(a_mn), int(b_mn), bias, aux, aux_out, out, flags, 1.0, M, N, K, self.ws.peer_ptrs_dev, self.own_base,
            self.ws.mc_ptr if self.use_multimem else 0, data_off, flag_off, _FLAG_BYTES, self.rank, self.world,
            epoch, self.done_totals[slot] & 0xFFFFFFFF, mode, self.use_multimem, self.trace)
        self.done_totals[slot] += int(inc)
        return data_off

    def gemm_all_reduce(self, a: Tensor, b: Tensor, a_mn: bool, b_mn: bool, partial: Optional[Tensor] = None,
                        copy: bool = True) -> Tensor:
        """``sum over ranks of (a @ b^T + partial)`` as ``[M, N]``: a fresh tensor, or with ``copy=False`` a view of
        the workspace slot that must be consumed before ``N_SLOTS - 1`` further fused calls are issued.
        ``partial`` is another per-rank partial sum ``[M, N]`` that joins this rank's tiles before the reduction."""
        M = a.size(1) if a_mn else a.size(0)
        K = a.size(0) if a_mn else a.size(1)
        N = b.size(1) if b_mn else b.size(0)
        off = self._call(a, b, a_mn, b_mn, None, None, None, _FLAG_RESIDUAL if partial is not None else 0, M, N, K,
                         MODE_ALLREDUCE, aux=partial)
        view = self.ws.buf.view(torch.uint8)[off: off + M * N * 2].view(a.dtype).view(M, N)
        return view.clone() if copy else view

    def gemm_reduce_scatter(self, a: Tensor, b: Tensor, a_mn: bool, b_mn: bool, partial: Optional[Tensor] = None) -> Tensor:
        M = a.size(1) if a_mn else a.size(0)
        K = a.size(0) if a_mn else a.size(1)
        N = b.size(1) if b_mn else b.size(0)
        out = torch.empty(M // self.world, N, dtype=a.dtype, device=a.device)
        self._call(a, b, a_mn, b_mn, None, None, out, _FLAG_RESIDUAL if partial is not None else 0, M, N, K,
                   MODE_REDUCE_SCATTER, aux=partial)
        return out

    def all_gather_gemm(self, a_shard: Tensor, b: Tensor, b_mn: bool, bias: Optional[Tensor] = None,
                        gelu: bool = False, save_preact: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        """Returns ``(product [M, N], gathered a [M, K])``; the gathered operand is a copy out of the workspace
        that the backward pass reuses for the weight gradient."""
        rows, K = a_shard.shape
        M = rows * self.world
        N = b.size(1) if b_mn else b.size(0)
        out = torch.empty(M, N, dtype=a_shard.dtype, device=a_shard.device)
        flags = (1 if bias is not None else 0) | (2 if gelu else 0) | (4 if save_preact is not None else 0)
        off = self._call(a_shard, b, False, b_mn, bias, save_preact, out, flags, M, N, K, MODE_ALLGATHER)
        gathered = self.ws.buf.view(torch.uint8)[off: off + M * K * 2].view(a_shard.dtype).view(M, K).clone()
        return out, gathered


def get_fused_tp(group) -> FusedTP:
    name = group.group_name
    ctx = _CONTEXTS.get(name)
    if ctx is None:
        ctx = FusedTP(group)
        _CONTEXTS[name] = ctx
    return ctx


def fused_tp_usable(mpu, x: Tensor, n_out: int, rows: Optional[int] = None) -> bool:
    """Fused paths need CUDA, the extension, 16-bit inputs, 8-aligned dims and a workspace slot that holds [M, N]."""
    if mpu is None or mpu.tp == 1 or not x.is_cuda or mpu.backend != "nccl" or not get_config().fused_tp_comm:
        return False
    if x.dtype not in (torch.bfloat16, torch.float16) or x.size(-1) % 8 or n_out % 8 or x.numel() == 0:
        return False
    if not ops.kernels_available() or not group_on_one_node(mpu.get_tensor_parallel_group()):
        return False
    rows = rows if rows is not None else x.numel() // x.size(-1)
    # decode-sized inputs gain nothing from overlapping tiles with their transfer, and the kernels take their
    # generation numbers as launch arguments, which a replayed CUDA graph would freeze: such calls use the plain
    # GEMM followed by the one-shot symmetric-memory all-reduce instead
    if rows < 128 or torch.cuda.is_current_stream_capturing():
        return False
    ctx = get_fused_tp(mpu.get_tensor_parallel_group())
    return ctx.fits(rows, max(n_out, x.size(-1)))  # forward and backward staging matrices


class _RowParallelFused(torch.autograd.Function):
    """``y = all_reduce(x_shard @ W_shard^T)``; backward needs no communication."""

    @staticmethod
    def forward(ctx, x, weight, reversed_, tp: FusedTP, partial=None, copy=True):
        """``partial``: this rank's partial sum of another row-parallel product with the same output shape; it joins
        the tiles before the reduction, so both products share the one all-reduce. ``copy=False``: the result is a
        view of the workspace (the caller consumes it at once, e.g. by adding the bias)."""
        x2 = x.reshape(-1, x.size(-1))
        p2 = None
        if partial is not None:
            p2 = partial.reshape(x2.size(0), -1)
            if p2.stride(-1) != 1:
                p2 = p2.contiguous()
        y = tp.gemm_all_reduce(x2, weight, False, reversed_, partial=p2, copy=copy)
        ctx.save_for_backward(x2, weight)
        ctx.reversed, ctx.in_shape = reversed_, x.shape
        ctx.partial_shape = partial.shape if partial is not None else None
        return y.view(*x.shape[:-1], y.size(-1))

    @staticmethod
    def backward(ctx, dy):
        from ..ops.cuda_ops import gemm, weight_grad
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, False, not ctx.reversed).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = weight_grad(weight, x2, dy2) if ctx.reversed else weight_grad(weight, dy2, x2)
        d_partial = dy.reshape(ctx.partial_shape) if (ctx.partial_shape is not None and ctx.needs_input_grad[4]) else None
        return dx, dw, None, None, d_partial, None


class _ColumnParallelFused(torch.autograd.Function):
    """``y = act(x @ W_shard^T + b)`` with a replicated ``x``; the input gradient ``sum_r dy_r W_r`` is one
    GEMM + all-reduce kernel (the reference's ``Broadcast.backward`` all-reduce)."""

    @staticmethod
    def forward(ctx, x, weight, bias, reversed_, gelu, tp: FusedTP):
        from ..ops.cuda_ops import FLAG_BIAS, FLAG_GELU, FLAG_SAVE_PREACT, gemm
        x2 = x.reshape(-1, x.size(-1))
        n = weight.size(1) if reversed_ else weight.size(0)
        flags = (FLAG_BIAS if bias is not None else 0) | (FLAG_GELU if gelu else 0)
        z = None
        if gelu and any(ctx.needs_input_grad[:3]):
            flags |= FLAG_SAVE_PREACT
            z = torch.empty(x2.size(0), n, dtype=x.dtype, device=x.device)
        y = gemm(x2, weight, False, reversed_, bias=bias, aux_out=z, flags=flags)
        ctx.save_for_backward(x2, weight, z)
        ctx.reversed, ctx.in_shape, ctx.tp = reversed_, x.shape, tp
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return y.view(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.cuda_ops import gemm, weight_grad
        ext = ops.load_ext(required=True)
        x2, weight, z = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if z is not None:
            dy2 = ext.bias_gelu_bwd(dy2, z, None)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # the input gradient goes straight to the next backward node (or is summed, out of place, with the
            # residual branch's gradient): a view of the workspace slot is enough
            dx = ctx.tp.gemm_all_reduce(dy2, weight, False, not ctx.reversed, copy=False).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = weight_grad(weight, x2, dy2) if ctx.reversed else weight_grad(weight, dy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ext.colsum(dy2).to(ctx.bias_dtype)
        return dx, dw, db, None, None, None


class _ColumnParallelSeqFused(torch.autograd.Function):
    """Sequence-parallel column layer: forward = all-gather(x) fused into the GEMM, backward input gradient =
    GEMM fused with the reduce-scatter."""

    @staticmethod
    def forward(ctx, x_shard, weight, bias, reversed_, gelu, tp: FusedTP):
        x2 = x_shard.reshape(-1, x_shard.size(-1))
        n = weight.size(1) if reversed_ else weight.size(0)
        z = None
        if gelu and any(ctx.needs_input_grad[:3]):
            z = torch.empty(x2.size(0) * tp.world, n, dtype=x2.dtype, device=x2.device)
        y, gathered = tp.all_gather_gemm(x2.contiguous(), weight, reversed_, bias, gelu, z)
        ctx.save_for_backward(gathered, weight, z)
        ctx.reversed, ctx.tp = reversed_, tp
        ctx.shard_shape = x_shard.shape
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        lead = list(x_shard.shape[:-1])
        lead[-1] *= tp.world  # the gathered (second to last) dim is the sequence
        return y.view(*lead, n)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.cuda_ops import gemm, weight_grad
        ext = ops.load_ext(required=True)
        gathered, weight, z = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if z is not None:
            dy2 = ext.bias_gelu_bwd(dy2, z, None)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = ctx.tp.gemm_reduce_scatter(dy2, weight, False, not ctx.reversed).view(ctx.shard_shape)
        if ctx.needs_input_grad[1]:
            dw = weight_grad(weight, gathered, dy2) if ctx.reversed else weight_grad(weight, dy2, gathered)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ext.colsum(dy2).to(ctx.bias_dtype)
        return dx, dw, db, None, None, None


class _RowParallelSeqFused(torch.autograd.Function):
    """Sequence-parallel row layer: forward = GEMM fused with the reduce-scatter, backward = all-gather(dy)
    fused into both gradient GEMMs' producer."""

    @staticmethod
    def forward(ctx, x, weight, reversed_, tp: FusedTP, partial=None):
        """``partial``: another row-parallel layer's partial sum over the same (gathered) rows; it joins this rank's
        tiles before the reduce-scatter."""
        x2 = x.reshape(-1, x.size(-1))
        p2 = None
        if partial is not None:
            p2 = partial.reshape(x2.size(0), -1)
            if p2.stride(-1) != 1:
                p2 = p2.contiguous()
        y = tp.gemm_reduce_scatter(x2, weight, False, reversed_, partial=p2)
        ctx.save_for_backward(x2, weight)
        ctx.reversed, ctx.tp, ctx.in_shape = reversed_, tp, x.shape
        ctx.partial_shape = partial.shape if partial is not None else None
        lead = list(x.shape[:-1])
        lead[-1] //= tp.world
        return y.view(*lead, y.size(-1))

    @staticmethod
    def backward(ctx, dy_shard):
        from ..ops.cuda_ops import gemm, weight_grad
        x2, weight = ctx.saved_tensors
        d2 = dy_shard.reshape(-1, dy_shard.size(-1)).contiguous()
        dx = dw = None
        # dx = all_gather(dy) @ W : the gathered dy comes back as a by-product and feeds the weight gradient
        dx2, dy_full = ctx.tp.all_gather_gemm(d2, weight, not ctx.reversed)
        if ctx.needs_input_grad[0]:
            dx = dx2.view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = weight_grad(weight, x2, dy_full) if ctx.reversed else weight_grad(weight, dy_full, x2)
        d_partial = None
        if ctx.partial_shape is not None and ctx.needs_input_grad[4]:
            d_partial = dy_full.reshape(ctx.partial_shape)      # backward of a reduce-scatter is the all-gather
        return dx, dw, None, None, d_partial


class _TPBlockInput(torch.autograd.Function):
    """The four column-parallel layers of a GPT-J block that read the same LayerNorm output - q, k, v and
    fc_in (+ tanh-GeLU) - as ONE autograd node under tensor parallelism.

    Forward is four local GEMMs. The point is the backward: the reference all-reduces the input gradient of every
    column-parallel layer separately (oslo/parallelism/mpu.py:848-856, four collectives per block); here the three
    short q / k / v products accumulate into one partial sum in their GEMM epilogues and that partial sum rides along
    in the epilogue of fc_in's long GEMM + all-reduce kernel, so the block's input gradient costs ONE collective,
    hidden behind the longest of the four products. Without the kernels (CPU / gloo) the same sum is formed with
    library matmuls and reduced once.
    """

    @staticmethod
    def forward(ctx, x, wq, wk, wv, w_in, b_in, mpu):
        on_gpu = x.is_cuda
        k = x.size(-1)
        x2 = x.reshape(-1, k)
        need_grad = any(ctx.needs_input_grad[:6])
        outs = []
        z = None
        if on_gpu:
            from ..ops.cuda_ops import FLAG_BIAS, FLAG_GELU, FLAG_SAVE_PREACT, gemm
            for w in (wq, wk, wv):
                y = torch.empty(*x.shape[:-1], w.size(0), dtype=x.dtype, device=x.device)
                gemm(x2, w, False, False, out=y.view(-1, w.size(0)))
                outs.append(y)
            flags = FLAG_GELU | (FLAG_BIAS if b_in is not None else 0)
            if need_grad:
                flags |= FLAG_SAVE_PREACT
                z = torch.empty(x2.size(0), w_in.size(0), dtype=x.dtype, device=x.device)
            h = torch.empty(*x.shape[:-1], w_in.size(0), dtype=x.dtype, device=x.device)
            gemm(x2, w_in, False, False, bias=b_in, out=h.view(-1, w_in.size(0)), aux_out=z, flags=flags)
        else:
            for w in (wq, wk, wv):
                outs.append((x2 @ w.t()).view(*x.shape[:-1], w.size(0)))
            z = x2 @ w_in.t()
            if b_in is not None:
                z = z + b_in
            h = ops.reference.gelu_tanh(z).to(x.dtype).view(*x.shape[:-1], w_in.size(0))
        ctx.save_for_backward(x2, wq, wk, wv, w_in, z)
        ctx.mpu, ctx.in_shape, ctx.has_bias = mpu, x.shape, b_in is not None
        ctx.fused = bool(on_gpu and fused_tp_usable(mpu, x, k))
        return outs[0], outs[1], outs[2], h

    @staticmethod
    def backward(ctx, dq, dk, dv, dh):
        x2, wq, wk, wv, w_in, z = ctx.saved_tensors
        mpu = ctx.mpu
        on_gpu = x2.is_cuda
        rows = x2.size(0)

        def flat(t):
            t = t.reshape(rows, -1)
            return t if t.is_contiguous() else t.contiguous()

        grads = [flat(d) if d is not None else None for d in (dq, dk, dv)]
        dh2 = flat(dh) if dh is not None else None
        dws = [None, None, None]
        dw_in = db_in = dx = None
        if on_gpu:
            from ..ops.cuda_ops import FLAG_ACCUMULATE, gemm, weight_grad
            ext = ops.load_ext(required=True)
            dz = ext.bias_gelu_bwd(dh2, z, None) if dh2 is not None else None
            part = None
            if ctx.needs_input_grad[0]:
                for d, w in zip(grads, (wq, wk, wv)):
                    if d is None:
                        continue
                    if part is None:
                        part = gemm(d, w, False, True)
                    else:
                        gemm(d, w, False, True, out=part, flags=FLAG_ACCUMULATE)
                if dz is not None and ctx.fused:
                    tp = get_fused_tp(mpu.get_tensor_parallel_group())
                    dx = tp.gemm_all_reduce(dz, w_in, False, True, partial=part, copy=False)      # the one collective
                else:
                    if dz is not None:
                        if part is None:
                            part = gemm(dz, w_in, False, True)
                        else:
                            gemm(dz, w_in, False, True, out=part, flags=FLAG_ACCUMULATE)
                    dx = mpu._reduce(part) if (mpu is not None and mpu.tp > 1) else part
            for i, (d, w) in enumerate(zip(grads, (wq, wk, wv))):
                if d is not None and ctx.needs_input_grad[1 + i]:
                    dws[i] = weight_grad(w, d, x2)
            if dz is not None and ctx.needs_input_grad[4]:
                dw_in = weight_grad(w_in, dz, x2)
            if dz is not None and ctx.has_bias and ctx.needs_input_grad[5]:
                db_in = ext.colsum(dz).to(dh.dtype)
        else:
            dz = None
            if dh2 is not None:
                zf = z.detach().float().requires_grad_(True)
                with torch.enable_grad():
                    ops.reference.gelu_tanh(zf).backward(dh2.float())
                dz = zf.grad.to(x2.dtype)
            if ctx.needs_input_grad[0]:
                part = None
                for d, w in zip(grads + [dz], (wq, wk, wv, w_in)):
                    if d is not None:
                        part = d @ w if part is None else part + d @ w
                dx = mpu._reduce(part) if (mpu is not None and mpu.tp > 1) else part
            for i, (d, w) in enumerate(zip(grads, (wq, wk, wv))):
                if d is not None and ctx.needs_input_grad[1 + i]:
                    dws[i] = d.t() @ x2
            if dz is not None and ctx.needs_input_grad[4]:
                dw_in = dz.t() @ x2
            if dz is not None and ctx.has_bias and ctx.needs_input_grad[5]:
                db_in = dz.sum(0)
        return (dx.view(ctx.in_shape) if dx is not None else None, dws[0], dws[1], dws[2], dw_in, db_in, None)


def tp_block_input(x: Tensor, wq: Tensor, wk: Tensor, wv: Tensor, w_in: Tensor, b_in: Optional[Tensor], mpu):
    """``(q, k, v, gelu(fc_in(x)))`` for column-parallel weight shards ``[out_shard, in]``; see ``_TPBlockInput``."""
    return _TPBlockInput.apply(x, wq, wk, wv, w_in, b_in, mpu)
