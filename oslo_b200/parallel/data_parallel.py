"""Data parallelism: bucketed gradient reduction over the data-parallel group, overlapped with backward
and aware of micro-batches.

The reference has no gradient code of its own: users wrap ``model.gpu_modules()`` in torch DDP or
DeepSpeed with ``process_group=model.mpu.get_data_parallel_group()`` (USAGE.md:128-155), and under
pipeline parallelism torch DDP only reduces the first micro-batch's backward. This wrapper

* keeps gradients in one flat buffer cut into buckets in reverse parameter order,
* reduces a bucket as soon as every gradient of the bucket has been accumulated - but only during the
  backward of the LAST micro-batch of a step (earlier micro-batches accumulate locally), so the reduction
  overlaps that backward and runs once per step. On GPUs the flat buffers live in symmetric memory and the
  reduction is this package's reduce-scatter kernel on a side stream (``csrc/comm.cu``; followed by the
  all-gather kernel when the optimizer state is not sharded); elsewhere it is an asynchronous all-reduce,
* hands the summed gradients to the optimizer, which divides by the group size (``FusedAdamW`` then only
  steps its shard),
* with ZeRO-1 sends the refreshed parameters out bucket by bucket under the next forward pass: every forward
  unit waits for the buckets that hold its own parameters only.

``torch.nn.parallel.DistributedDataParallel`` around ``gpu_modules()`` keeps working for steps that
have a single micro-batch.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import get_config
from ..optim import FlatBuffers, FusedAdamW
from .mpu import MPU


def forward_units(root: nn.Module) -> List[nn.Module]:
    """The modules of ``root`` whose calls, in forward order, touch every parameter exactly at unit granularity: the
    items of ``nn.ModuleList`` containers (transformer blocks, pipeline-stage items) and, outside of them, every
    module that owns parameters directly (embeddings, the final norm, the head)."""
    units: List[nn.Module] = []

    def walk(m: nn.Module, in_list: bool) -> None:
        if in_list or (m._parameters and any(p is not None for p in m._parameters.values())):
            units.append(m)
            return
        for child in m.children():
            walk(child, isinstance(m, nn.ModuleList))

    walk(root, False)
    return units


class DistributedDataParallel(nn.Module):
    def __init__(self, model: nn.Module, mpu: MPU, optimizer: Optional[FusedAdamW] = None,
                 bucket_mb: float = 256.0, num_micro_batches: Optional[int] = None) -> None:
        super().__init__()
        self.module = model
        self.mpu = mpu
        self.group = mpu.get_data_parallel_group()
        self.world = mpu.get_data_parallel_world_size()
        self.optimizer = optimizer
        gm = model.gpu_modules() if hasattr(model, "gpu_modules") else model
        self.buf = optimizer.buf if optimizer is not None else FlatBuffers(gm.parameters(), symmetric_group=self.group)
        # buffers in symmetric memory: the bucket reductions are this package's reduce-scatter kernel on a side stream
        # (followed by the all-gather kernel where every rank needs the whole sum); otherwise NCCL all-reduce
        self._symm = self.buf.symm_g is not None and self.buf.symm_g.group is self.group
        self._zero = (optimizer is not None and optimizer.shards > 1 and optimizer.shard_group is self.group)
        self._side = torch.cuda.Stream() if self._symm else None
        self.sync = True
        self._pending: List = []
        self._ready: List[int] = []
        self._bucket_of = {}
        self.buckets: List[tuple] = []
        self._build_buckets(int(bucket_mb * 2 ** 20))
        for p in self.buf.params:
            p.register_post_accumulate_grad_hook(self._hook)
            p._oslo_grad_hook = self._hook   # called by weight-gradient GEMMs that add straight into p.grad
        eng = getattr(model, "_pipe_engine", None)
        self._deferred = set()
        if eng is not None:
            eng.on_last_backward = lambda last: setattr(self, "sync", bool(last))
            self._pipelined = True
            # an embedding tied between the first and the last stage is summed over those two stages AFTER the last
            # backward (engine_pipeline._allreduce_tied_embedding), in place, in this very buffer: its bucket must not
            # be in flight then, so it is reduced from finish_gradient_sync() instead of from the hook
            tied = (eng.pp > 1 and (eng.first or eng.last) and getattr(model.config, "tie_word_embeddings", True)
                    and model.get_output_embeddings() is not None)
            if tied:
                self._deferred.add(id(model.get_input_embeddings().weight))
        else:
            self._pipelined = False
        self._param_events: List = []
        self._param_pending: set = set()
        if (self._symm and self._zero and self.buf.symm_p is not None
                and get_config().dp_overlap_param_gather):
            self._install_param_gather(gm, optimizer)
        if optimizer is not None:
            optimizer.grads_already_reduced = True
            # the buckets are SUMMED over this group; the optimizer turns the sum into the mean (1 / group size), also
            # when its state is not sharded
            optimizer.grad_average_group = self.group
            self._wrap_optimizer_step(optimizer)

    # ------------------------------------------------------------------ buckets
    def _build_buckets(self, bucket_bytes: int) -> None:
        esize = self.buf.flat_g.element_size()
        params, offsets = self.buf.params, self.buf.offsets
        end = self.buf.padded
        cur: List[int] = []
        hi = end
        # walk parameters from the last (its gradient is produced first in backward) to the first
        for idx in range(len(params) - 1, -1, -1):
            cur.append(idx)
            lo = offsets[idx]
            if (hi - lo) * esize >= bucket_bytes or idx == 0:
                b = len(self.buckets)
                self.buckets.append((lo, hi, list(cur)))
                for i in cur:
                    self._bucket_of[id(params[i])] = b
                self._ready.append(0)
                cur, hi = [], lo

    def _hook(self, p: torch.Tensor) -> None:
        g = p.grad
        if g is not None and g.untyped_storage().data_ptr() != self.buf.flat_g.untyped_storage().data_ptr():
            # something (a torch optimizer's zero_grad(set_to_none=True)) dropped the view into the flat buffer and
            # autograd made a fresh tensor: a dropped gradient counts as zero, so the fresh one replaces the stale
            # contents of the view, and later micro-batches accumulate into the view again
            view = self._grad_view(p)
            view.copy_(g)
            p.grad = view
        if not self.sync or self.world == 1 or id(p) in self._deferred:
            return
        b = self._bucket_of[id(p)]
        self._ready[b] += 1
        if self._ready[b] == len(self.buckets[b][2]):
            self._launch(b)

    def _grad_view(self, p: torch.Tensor) -> torch.Tensor:
        if not hasattr(self, "_offset_of"):
            self._offset_of = {id(q): off for q, off in zip(self.buf.params, self.buf.offsets)}
        off = self._offset_of[id(p)]
        return self.buf.flat_g[off: off + p.numel()].view(p.shape)

    def _launch(self, b: int) -> None:
        lo, hi, _ = self.buckets[b]
        self._ready[b] = -(10 ** 9)  # launched
        if self._symm:
            # the bucket is complete at this point of the compute stream; everything else happens on the side stream
            self._side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side):
                self.buf.symm_g.reduce_scatter_(lo, hi)
                if not self._zero:
                    self.buf.symm_g.all_gather_(lo, hi)      # every rank steps every parameter: spread the sums
            return
        chunk = self.buf.flat_g[lo:hi]
        self._pending.append(dist.all_reduce(chunk, group=self.group, async_op=True))

    def finish_gradient_sync(self) -> None:
        """Wait for the bucket reductions of this step; launches any bucket that never became ready
        (parameters without gradient this step) so every rank issues the same collectives."""
        self.finish_param_sync()     # nothing is pending after a whole forward pass; a step without one gets here
        if self.world > 1:
            for b in range(len(self.buckets)):
                if self._ready[b] >= 0:
                    self._launch(b)
            for w in self._pending:
                w.wait()
            if self._symm:
                torch.cuda.current_stream().wait_stream(self._side)
            if self.optimizer is None:
                self.buf.flat_g.div_(self.world)
        self._pending = []
        self._ready = [0] * len(self.buckets)

    # ------------------------------------------------------------------ ZeRO-1 parameter all-gather, overlapped
    def _install_param_gather(self, gm: nn.Module, opt: FusedAdamW) -> None:
        """After the optimizer step the refreshed parameters of every shard travel bucket by bucket, in the order in
        which the forward pass needs them, on the side stream; every forward unit (an embedding, a transformer block,
        the final norm, the head) makes the compute stream wait for the buckets that hold its own parameters only.
        The first layers of the next step therefore start while the later layers' parameters are still in flight."""
        self._param_events = [torch.cuda.Event() for _ in self.buckets]
        units = forward_units(gm)
        for m in units:
            need = sorted({self._bucket_of[id(p)] for p in m.parameters() if id(p) in self._bucket_of}, reverse=True)
            if need:
                m.register_forward_pre_hook(self._make_unit_hook(need))
        covered = {id(p) for m in units for p in m.parameters()}
        if any(id(p) not in covered for p in self.buf.params):
            raise RuntimeError("a parameter belongs to no forward unit")    # cannot happen by construction
        # checkpoints read the parameters without running a forward pass: wait for every bucket first. Under pipeline
        # parallelism the stage module is not a registered child of the model, so both get the hook.
        for m in {id(x): x for x in (gm, self.module)}.values():
            m.register_state_dict_pre_hook(lambda *a, **k: self.finish_param_sync())
        opt.param_gather = self._gather_params

    def _gather_params(self) -> None:
        self._side.wait_stream(torch.cuda.current_stream())          # the optimizer step wrote this rank's shard
        with torch.cuda.stream(self._side):
            for b in range(len(self.buckets) - 1, -1, -1):           # bucket 0 holds the LAST parameters
                lo, hi, _ = self.buckets[b]
                self.buf.symm_p.all_gather_(lo, hi)
                self._param_events[b].record(self._side)
        self._param_pending = set(range(len(self.buckets)))

    def _make_unit_hook(self, need: List[int]):
        def hook(_module, _args):
            if self._param_pending:
                cur = torch.cuda.current_stream()
                for b in need:
                    if b in self._param_pending:
                        cur.wait_event(self._param_events[b])
                        self._param_pending.discard(b)
        return hook

    def finish_param_sync(self) -> None:
        """Make the current stream wait for every parameter bucket that is still in flight (before anything other
        than a forward pass reads the parameters: checkpoints, evaluation code that bypasses the modules)."""
        if self._param_pending:
            cur = torch.cuda.current_stream()
            for b in sorted(self._param_pending):
                cur.wait_event(self._param_events[b])
            self._param_pending = set()

    def _wrap_optimizer_step(self, opt: FusedAdamW) -> None:
        inner = opt.step
        ddp = self

        def step():
            ddp.finish_gradient_sync()
            return inner()

        opt.step = step

    # ------------------------------------------------------------------ module API
    @contextmanager
    def no_sync(self):
        """Accumulate gradients locally (use for every micro-batch of a step except the last)."""
        prev = self.sync
        self.sync = False
        try:
            yield
        finally:
            self.sync = prev

    def forward(self, *args, **kwargs):
        if self._pipelined:
            self.sync = False  # the pipeline engine switches it on for the last micro-batch
        return self.module(*args, **kwargs)

    def gpu_modules(self):
        return self.module.gpu_modules()

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)
