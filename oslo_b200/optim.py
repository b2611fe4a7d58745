"""Fused AdamW on flat buffers with fp32 master weights, optionally sharded over the data-parallel
group (ZeRO stage 1).

The reference leaves optimisation to ``torch.optim.Adam`` or DeepSpeed ZeRO wrapped around
``model.gpu_modules()`` (USAGE.md:128-155, :366-387). Here the same role is played natively:

* all parameters of a dtype live in one flat low-precision buffer (``param.data`` are views) and all
  gradients in one flat buffer (``param.grad`` are views), so a step is ONE kernel launch and a
  data-parallel reduction is a handful of large collectives instead of one per tensor;
* master weights and both moments are fp32; the kernel writes the refreshed bf16/fp16 copy;
* with ``shard_group`` every rank keeps master/moments for ``1/dp`` of the flat buffer only:
  gradients are reduce-scattered, the owned shard is stepped, parameters are all-gathered;
* gradient clipping uses a device-side norm, no host synchronisation;
* fp16 training: ``DynamicLossScaler`` (the role DeepSpeed's fp16 optimizer or ``torch.cuda.amp.GradScaler``
  plays for the reference, USAGE.md:243-267, tests/gpt2/gpt2_test_3d_training.py ZeRO config): the overflow
  check reuses the norm reduction, so every data-, tensor- and pipeline-parallel rank takes the same decision.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from . import ops


def sync_sequence_parallel_grads(model) -> None:
    """Sum, over the tensor-parallel group, the gradients of parameters that a sequence-parallel model applies
    to a token shard (LayerNorm weights, row-parallel biases). ``FusedAdamW(model=...)`` does this itself;
    call it by hand before ``step()`` of any other optimizer."""
    params = [p for p in (getattr(model, "_sp_partial_params", None) or []) if p.grad is not None]
    if not params:
        return
    flat = torch.cat([p.grad.reshape(-1) for p in params])
    dist.all_reduce(flat, group=model.mpu.get_tensor_parallel_group())
    off = 0
    for p in params:
        p.grad.copy_(flat[off: off + p.numel()].view_as(p.grad))
        off += p.numel()


class DynamicLossScaler:
    """Loss scale for fp16 gradients: halve on overflow (and skip that step), double after
    ``growth_interval`` clean steps. bf16 training does not need one."""

    def __init__(self, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, min_scale: float = 1.0, max_scale: float = 2.0 ** 24) -> None:
        if not (growth_factor > 1.0 and 0.0 < backoff_factor < 1.0 and growth_interval > 0 and init_scale > 0):
            raise ValueError("need growth_factor > 1, 0 < backoff_factor < 1, growth_interval > 0, init_scale > 0")
        self.loss_scale = float(init_scale)
        self.growth_factor, self.backoff_factor = float(growth_factor), float(backoff_factor)
        self.growth_interval = int(growth_interval)
        self.min_scale, self.max_scale = float(min_scale), float(max_scale)
        self.good_steps = 0
        self.skipped_steps = 0

    def scale(self, loss: Tensor) -> Tensor:
        """``scaler.scale(loss).backward()``; pipeline stages without the head scale a proxy whose gradient
        arrives already scaled from the next stage."""
        return loss * self.loss_scale

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self.loss_scale = max(self.loss_scale * self.backoff_factor, self.min_scale)
            self.good_steps = 0
            self.skipped_steps += 1
            return
        self.good_steps += 1
        if self.good_steps >= self.growth_interval:
            self.loss_scale = min(self.loss_scale * self.growth_factor, self.max_scale)
            self.good_steps = 0

    def state_dict(self) -> Dict[str, float]:
        return dict(loss_scale=self.loss_scale, good_steps=self.good_steps, skipped_steps=self.skipped_steps)

    def load_state_dict(self, sd: Dict[str, float]) -> None:
        self.loss_scale = float(sd["loss_scale"])
        self.good_steps = int(sd["good_steps"])
        self.skipped_steps = int(sd.get("skipped_steps", 0))


class FlatBuffers:
    """One flat parameter buffer + one flat gradient buffer per dtype; tensors become views.

    ``grad_dtype=torch.float32`` with 16-bit parameters keeps the gradient buffer in fp32 (main gradients): the
    micro-batch gradients of a step then accumulate without 16-bit rounding, at the price of twice the gradient bytes
    in memory and on the data-parallel wire, an extra pass per weight gradient (the 16-bit product is added into the
    fp32 buffer by autograd instead of inside the GEMM epilogue) and NCCL instead of the symmetric-memory kernels,
    which reduce 16-bit buffers. The default (gradients in the parameters' dtype) is what the benchmarks run."""

    def __init__(self, params: Iterable[torch.nn.Parameter], pad_to: int = 1, grad_dtype: Optional[torch.dtype] = None,
                 symmetric_group=None):
        """``symmetric_group``: keep both buffers in symmetric memory of this (data-parallel) group when the device and
        dtypes allow it (``parallel.symmetric.symmetric_flat_usable``), so gradient reduction and parameter
        all-gather can run as this package's kernels; collective over the group."""
        self.params: List[torch.nn.Parameter] = []
        seen = set()
        for p in params:
            if p.requires_grad and id(p) not in seen and p.numel() > 0:
                seen.add(id(p))
                self.params.append(p)
        if not self.params:
            raise ValueError("no trainable parameters")
        dts = {p.dtype for p in self.params}
        if len(dts) != 1:
            raise ValueError(f"parameters must share one dtype, got {dts}")
        self.dtype = self.params[0].dtype
        self.device = self.params[0].device
        self.offsets: List[int] = []
        n = 0
        for p in self.params:
            self.offsets.append(n)
            n += (p.numel() + 7) // 8 * 8  # keep every tensor 16-byte aligned for vector / TMA access
        self.numel = n
        self.padded = (n + pad_to - 1) // pad_to * pad_to
        self.symm_p = self.symm_g = None
        if symmetric_group is not None:
            from .parallel.symmetric import SymmetricFlat, symmetric_flat_usable
            if (symmetric_flat_usable(symmetric_group, self.dtype, self.device)
                    and (grad_dtype or self.dtype) == self.dtype):
                self.symm_p = SymmetricFlat(symmetric_group, self.padded, self.dtype, self.device)
                self.symm_g = SymmetricFlat(symmetric_group, self.padded, self.dtype, self.device)
        if self.symm_p is not None:
            self.flat_p, self.flat_g = self.symm_p.tensor, self.symm_g.tensor
        else:
            self.flat_p = torch.zeros(self.padded, dtype=self.dtype, device=self.device)
            self.flat_g = torch.zeros(self.padded, dtype=grad_dtype or self.dtype, device=self.device)
        wide = self.flat_g.dtype != self.dtype
        if wide and not hasattr(torch.Tensor, "grad_dtype"):
            raise RuntimeError("gradients in a dtype other than the parameters' need torch's Tensor.grad_dtype")
        for p, off in zip(self.params, self.offsets):
            view = self.flat_p[off: off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            if getattr(p, "grad_dtype", self.flat_g.dtype) != self.flat_g.dtype:
                # `grad_dtype` is what autograd converts incoming gradients to and accumulates in: with an fp32 buffer
                # the micro-batch gradients of 16-bit parameters add up in fp32. (Also the way back: a parameter that
                # an earlier buffer had switched to fp32 gradients.) The attribute only changes while .grad is unset.
                p.grad = None
                p.grad_dtype = self.flat_g.dtype
            p.grad = self.flat_g[off: off + p.numel()].view(p.shape)
            # the view lives as long as the buffer and is zeroed every step: weight-gradient GEMMs may add into it
            p._oslo_accum_grad = self.flat_g.dtype == p.dtype and not getattr(p, "_oslo_shared", False)

    def zero_grad(self) -> None:
        self.flat_g.zero_()
        for p, off in zip(self.params, self.offsets):  # re-attach in case something set grads to None
            if p.grad is None or p.grad.data_ptr() != self.flat_g.data_ptr() + off * self.flat_g.element_size():
                p.grad = self.flat_g[off: off + p.numel()].view(p.shape)


class FusedAdamW:
    """AdamW with fp32 master weights on ``FlatBuffers``; ``shard_group`` turns on ZeRO-1 sharding."""

    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: Optional[float] = None, shard_group=None,
                 grad_average_group=None, model_parallel_group=None, model=None,
                 loss_scaler: Optional[DynamicLossScaler] = None, grad_dtype: Optional[torch.dtype] = None) -> None:
        self.lr, self.betas, self.eps, self.weight_decay = lr, tuple(betas), eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.loss_scaler = loss_scaler
        self.shard_group = shard_group
        self.model_parallel_group = model_parallel_group
        self.shards = dist.get_world_size(shard_group) if shard_group is not None else 1
        self.shard_rank = dist.get_rank(shard_group) if shard_group is not None else 0
        self.grad_average_group = grad_average_group
        # `params` is an iterable of parameters or, as with torch optimizers, a list of groups
        # ``{"params": [...], "weight_decay": 0.0, "lr": ...}``: the groups lie one after the other in the flat buffer
        params = list(params)
        if params and isinstance(params[0], dict):
            groups = [dict(g, params=list(g["params"])) for g in params]
        else:
            groups = [dict(params=params)]
        self.buf = FlatBuffers([p for g in groups for p in g["params"]], pad_to=8 * self.shards, grad_dtype=grad_dtype,
                               symmetric_group=shard_group if self.shards > 1 else grad_average_group)
        n = self.buf.padded // self.shards
        self.shard_numel = n
        lo = self.shard_rank * n
        self._lo, self._hi = lo, lo + n
        dev = self.buf.device
        self.master = self.buf.flat_p[lo: lo + n].float()
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.grads_already_reduced = False  # set by DistributedDataParallel, which all-reduces buckets itself
        self.param_gather = None            # set by DistributedDataParallel: how the refreshed parameters are spread
        # sequence parallelism: LayerNorm weights and row-parallel biases act on a token shard, so their
        # gradients must be summed over the tensor-parallel group before the update
        self._sp_params = list(getattr(model, "_sp_partial_params", []) or []) if model is not None else []
        self._sp_group = model.mpu.get_tensor_parallel_group() if self._sp_params else None
        # one entry per group, torch style (learning-rate schedulers write `param_groups[i]["lr"]`); `_group_ranges`
        # holds each group's part of this rank's shard, relative to the shard
        index = {id(p): i for i, p in enumerate(self.buf.params)}
        self.param_groups, self._group_ranges = [], []
        for g in groups:
            kept = [p for p in g["params"] if id(p) in index]
            self.param_groups.append(dict(params=kept, lr=g.get("lr", lr), betas=self.betas, eps=eps,
                                          weight_decay=g.get("weight_decay", weight_decay)))
        bounds, seen_ids = [], set()
        for g in self.param_groups:
            ids = [index[id(p)] for p in g["params"] if id(p) not in seen_ids]
            seen_ids.update(id(p) for p in g["params"])
            if ids and ids != list(range(ids[0], ids[-1] + 1)):
                raise ValueError("a parameter appears in more than one group")
            bounds.append((self.buf.offsets[ids[0]], None) if ids else None)
        starts = [b[0] for b in bounds if b is not None] + [self.buf.padded]
        k = 0
        for b in bounds:
            if b is None:
                self._group_ranges.append(None)
                continue
            a, e = max(starts[k], self._lo), min(starts[k + 1], self._hi)
            self._group_ranges.append((a - self._lo, e - self._lo) if e > a else None)
            k += 1
        # gradients that another model-parallel rank also holds (tensors replicated over the tensor-parallel group,
        # the last pipeline stage's copy of a tied embedding) count once in the global norm: the parts of them that
        # fall into this rank's shard are subtracted again
        self._dup_ranges: List[tuple] = []      # relative to this rank's shard of the flat buffer
        for p, off in zip(self.buf.params, self.buf.offsets):
            if getattr(p, "_oslo_norm_dup", False):
                a, b = max(off, self._lo), min(off + p.numel(), self._hi)
                if b > a:
                    self._dup_ranges.append((a - self._lo, b - self._lo))
        self._dup_cache = (None, [])            # (data_ptr of the gradient shard, its views)

    # ------------------------------------------------------------------ API
    def zero_grad(self, set_to_none: bool = False) -> None:
        self.buf.zero_grad()

    def grad_norm(self, g: Tensor) -> Tensor:
        """2-norm of the (sharded) gradient over all shards and model-parallel ranks, as a device scalar."""
        if g.is_cuda and ops.kernels_available():
            sq = ops.load_ext().sumsq(g)
        else:
            sq = g.float().pow(2).sum().reshape(1)
        if self._dup_ranges:
            if g.untyped_storage().data_ptr() != self.buf.flat_g.untyped_storage().data_ptr():
                views = [g[a:b] for a, b in self._dup_ranges]      # a temporary (reduce-scatter output): keep nothing
            else:
                if self._dup_cache[0] != g.data_ptr():
                    self._dup_cache = (g.data_ptr(), [g[a:b] for a, b in self._dup_ranges])
                views = self._dup_cache[1]
            dup = torch.stack(torch._foreach_norm(views, 2, dtype=torch.float32)).pow(2).sum()
            sq = (sq - dup).clamp_min(0.0)
        for grp in (self.shard_group, self.model_parallel_group):
            if grp is not None and dist.get_world_size(grp) > 1:
                dist.all_reduce(sq, group=grp)
        return sq.sqrt()

    def sync_sequence_parallel_grads(self) -> None:
        grads = [p.grad for p in self._sp_params if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=self._sp_group)
        off = 0
        for g in grads:
            g.copy_(flat[off: off + g.numel()].view_as(g))
            off += g.numel()

    @torch.no_grad()
    def step(self) -> bool:
        """One update; returns False when the loss scaler saw an overflow and the update was skipped."""
        self.sync_sequence_parallel_grads()
        b1, b2 = self.betas
        g_full = self.buf.flat_g
        if self.shards > 1 and self.grads_already_reduced:
            g = g_full[self._lo: self._hi]
            grad_scale = 1.0 / self.shards
        elif self.shards > 1 and self.buf.symm_g is not None:
            self.buf.symm_g.reduce_scatter_(0, self.buf.padded)      # in place: this rank's shard becomes the sum
            g = g_full[self._lo: self._hi]
            grad_scale = 1.0 / self.shards
        elif self.shards > 1:
            g = torch.empty(self.shard_numel, dtype=g_full.dtype, device=g_full.device)
            if dist.get_backend(self.shard_group) == "gloo":
                dist.all_reduce(g_full, group=self.shard_group)
                g.copy_(g_full[self._lo: self._hi])
            else:
                dist.reduce_scatter_tensor(g, g_full, group=self.shard_group)
            grad_scale = 1.0 / self.shards
        else:
            g = g_full
            grad_scale = 1.0
            if self.grads_already_reduced and self.grad_average_group is not None:
                # plain data parallelism (no sharded state): the wrapper summed the buckets, the mean is taken here
                grad_scale = 1.0 / dist.get_world_size(self.grad_average_group)
        inv = None
        norm = None
        if self.loss_scaler is not None:
            # the squared norm is summed over the shard and model-parallel groups, so every rank that shares
            # these parameters (or the loss) reads the same value and skips or steps together
            norm = self.grad_norm(g)
            found_inf = not bool(torch.isfinite(norm).item())
            if found_inf:
                self.loss_scaler.update(True)
                return False
            grad_scale /= self.loss_scaler.loss_scale
            self.loss_scaler.update(False)
        self.step_count += 1
        if self.max_grad_norm is not None:
            norm = (self.grad_norm(g) if norm is None else norm) * grad_scale
            inv = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0).float()
        lp = self.buf.flat_p[self._lo: self._hi]
        use_kernel = g.is_cuda and ops.kernels_available()
        scale = None if use_kernel else grad_scale * (float(inv) if inv is not None else 1.0)
        for group, rng in zip(self.param_groups, self._group_ranges):     # one launch per group (usually one or two)
            if rng is None:
                continue
            a, e = rng
            whole = a == 0 and e == self.shard_numel
            m_, g_, ea_, es_, lp_ = ((self.master, g, self.exp_avg, self.exp_avg_sq, lp) if whole else
                                     (self.master[a:e], g[a:e], self.exp_avg[a:e], self.exp_avg_sq[a:e], lp[a:e]))
            if use_kernel:
                ops.load_ext().adam_step(m_, g_, ea_, es_, lp_ if lp.dtype != torch.float32 else None, group["lr"],
                                         b1, b2, self.eps, group["weight_decay"], self.step_count, grad_scale, inv)
            else:
                ops.reference.adam_step(m_, g_, ea_, es_, self.step_count, group["lr"], b1, b2, self.eps,
                                        group["weight_decay"], scale, lp_)
        if use_kernel and lp.dtype == torch.float32:
            lp.copy_(self.master)
        if self.shards > 1 and self.buf.symm_p is not None:
            if self.param_gather is not None:
                self.param_gather()          # the data-parallel wrapper: bucket by bucket, overlapped with the forward
            else:
                self.buf.symm_p.all_gather_(0, self.buf.padded)
        elif self.shards > 1:
            if dist.get_backend(self.shard_group) == "gloo":
                parts = [torch.empty_like(lp) for _ in range(self.shards)]
                dist.all_gather(parts, lp.contiguous(), group=self.shard_group)
                self.buf.flat_p.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(self.buf.flat_p, lp.contiguous(), group=self.shard_group)
        return True

    # ------------------------------------------------------------------ checkpoint sidecar
    def state_dict(self) -> Dict[str, object]:
        return dict(step=self.step_count, master=self.master.cpu(), exp_avg=self.exp_avg.cpu(),
                    exp_avg_sq=self.exp_avg_sq.cpu(), shard_rank=self.shard_rank, shards=self.shards, lr=self.lr,
                    loss_scaler=self.loss_scaler.state_dict() if self.loss_scaler is not None else None,
                    group_lrs=[g["lr"] for g in self.param_groups])

    @staticmethod
    def reshard_state(states: List[Dict[str, object]], shards: int, shard_rank: int, shard_numel: int) -> Dict[str, object]:
        """The state of shard ``shard_rank`` of ``shards`` (``shard_numel`` elements each) cut out of the states that the
        ranks of ANOTHER data-parallel size saved: ZeRO-1 shards are consecutive slices of one flat buffer, so a job
        that continues with fewer or more replicas (same tensor / pipeline layout) re-cuts them. ``states`` may hold
        only the old shards that overlap the new one; what lies beyond the old buffer's padded end is padding here too."""
        if not states:
            raise ValueError("no optimizer states to re-cut")
        old = sorted(states, key=lambda s: int(s["shard_rank"]))
        n_old = old[0]["master"].numel()
        lo, hi = shard_rank * shard_numel, (shard_rank + 1) * shard_numel
        out = {k: torch.zeros(shard_numel, dtype=torch.float32) for k in ("master", "exp_avg", "exp_avg_sq")}
        covered = 0
        for s in old:
            if s["master"].numel() != n_old or int(s["shards"]) != int(old[0]["shards"]):
                raise ValueError("optimizer states of different shardings cannot be combined")
            a = int(s["shard_rank"]) * n_old
            x, y = max(a, lo), min(a + n_old, hi)
            if y > x:
                for k in out:
                    out[k][x - lo: y - lo] = s[k][x - a: y - a]
                covered += y - x
        need = max(0, min(hi, int(old[0]["shards"]) * n_old) - lo)
        if covered != need:
            raise ValueError(f"the given states cover {covered} of the {need} elements shard {shard_rank} needs")
        first = old[0]
        return dict(first, shard_rank=shard_rank, shards=shards, **out)

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        if sd["shards"] != self.shards or sd["shard_rank"] != self.shard_rank:
            raise ValueError("optimizer state was saved with a different sharding")
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.buf.flat_p[self._lo: self._hi].copy_(self.master)
        lrs = sd.get("group_lrs")
        if lrs is not None and len(lrs) == len(self.param_groups):
            for g, lr in zip(self.param_groups, lrs):     # where a schedule had brought each group
                g["lr"] = lr
        if self.loss_scaler is not None and sd.get("loss_scaler") is not None:
            self.loss_scaler.load_state_dict(sd["loss_scaler"])
