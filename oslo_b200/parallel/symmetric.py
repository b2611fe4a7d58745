"""Symmetric-memory workspace of one process group and the collectives that run on it.

Allocation and rendezvous (CUDA VMM handles exchanged between the ranks, peer mappings, the NVSwitch
multicast mapping and the signal pads) come from ``torch.distributed._symmetric_memory``; the device
protocol and the kernels are this package's own (``csrc/comm.cu``, ``csrc/fused_comm_gemm.cu``): they get
raw peer / multicast / signal-pad addresses and run the compare-and-swap handshake and the
``multimem`` loads and stores themselves.

A peer's memory is only ever touched by plain loads / stores or ``multimem`` instructions issued by these
kernels; it is never handed to a library kernel or to a TMA load.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..config import get_config

_WORKSPACES: Dict[str, "SymmetricWorkspace"] = {}
ONESHOT_HALF = 1 << 20   # bytes per staging half of the one-kernel all-reduce


_ONE_NODE: Dict[str, bool] = {}


def node_identity() -> str:
    """What two ranks must share to map each other's memory: the host (its name and the identifier of its current
    boot). ``OSLO_B200_NODE_ID`` overrides it (tests; clusters whose host names are not unique)."""
    import os
    import socket
    override = os.environ.get("OSLO_B200_NODE_ID")
    if override:
        return override
    boot = ""
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            boot = f.read().strip()
    except OSError:
        pass
    return f"{socket.gethostname()}|{boot}"


def remember_group_nodes(group, nodes) -> None:
    """Record the hosts of a group's ranks (the MPU knows them from its one exchange at construction)."""
    _ONE_NODE[group.group_name] = len(set(nodes)) == 1


def group_on_one_node(group) -> bool:
    """All ranks of ``group`` run on the same host. Symmetric memory (peer mappings, the NVSwitch multicast object)
    exists inside one NVLink domain only, so every path that uses it asks this first; a group that spans hosts stays
    on NCCL. Groups of an ``MPU`` are known from its construction; for any other group the first call is collective
    over the group (one small object all-gather), cached afterwards."""
    if group is None:
        return False
    name = group.group_name
    hit = _ONE_NODE.get(name)
    if hit is None:
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            return False          # no collective inside a stream capture; the caller falls back to NCCL this once
        n = dist.get_world_size(group)
        if n == 1:
            hit = True
        else:
            ids = [None] * n
            dist.all_gather_object(ids, node_identity(), group=group)
            hit = len(set(ids)) == 1
        _ONE_NODE[name] = hit
    return hit


class SymmetricWorkspace:
    def __init__(self, group, nbytes: int, device: Optional[torch.device] = None) -> None:
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.numel = (int(nbytes) + 255) // 256 * 128  # bf16 elements, 256-byte multiple
        self.buf = symm.empty(self.numel, dtype=torch.bfloat16, device=self.device)
        self.handle = symm.rendezvous(self.buf, group)
        self.peer_ptrs_dev = int(self.handle.buffer_ptrs_dev)
        self.signal_ptrs_dev = int(self.handle.signal_pad_ptrs_dev)
        self.signal_pad_bytes = int(self.handle.signal_pad_size)
        try:
            self.mc_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support else 0
        except Exception:
            self.mc_ptr = 0
        self.buf.zero_()
        # the last two ONESHOT_HALF-sized pieces of the buffer are the alternating staging halves of the
        # one-kernel all-reduce for small tensors; `oneshot_counters` holds their per-block parity on the device
        self.oneshot_half = ONESHOT_HALF if self.numel * 2 >= 4 * ONESHOT_HALF else 0
        self.oneshot_off = self.numel * 2 - 2 * self.oneshot_half
        self.oneshot_counters = torch.zeros(64, dtype=torch.int32, device=self.device)
        # the rest of the buffer, cut in two, stages the fused vocab-parallel embedding lookup
        self.embed_half = (self.oneshot_off // 2) // 256 * 256
        self.embed_counters = torch.zeros(64, dtype=torch.int32, device=self.device)
        self.handle.barrier()

    @property
    def has_multicast(self) -> bool:
        return self.mc_ptr != 0

    def view(self, numel: int, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        t = self.buf if dtype == torch.bfloat16 else self.buf.view(dtype)
        if numel > t.numel():
            raise ValueError(f"symmetric workspace too small: need {numel} elements, have {t.numel()}")
        return t[:numel]

    def all_reduce_(self, x: torch.Tensor, use_multimem: Optional[bool] = None) -> torch.Tensor:
        """Sum ``x`` (bf16 / fp16, numel % 8 == 0) over the group through the workspace; returns ``x``."""
        n = x.numel()
        if n % 8 or x.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("all_reduce_ needs a 16-bit tensor whose numel is a multiple of 8")
        if use_multimem is None:
            use_multimem = get_config().use_multimem
        use_multimem = bool(use_multimem) and self.has_multicast
        if self.oneshot_half and n * 2 <= self.oneshot_half and x.is_contiguous():
            ops.load_ext(required=True).allreduce_oneshot(x, self.peer_ptrs_dev, self.mc_ptr, self.signal_ptrs_dev,
                                                         self.oneshot_counters, self.oneshot_off, self.oneshot_half,
                                                         self.rank, self.world, use_multimem)
            return x
        if n * 2 > self.oneshot_off:
            raise ValueError("tensor does not fit the symmetric workspace")
        stage = self.view(n, x.dtype)
        flat = x.reshape(-1)
        stage.copy_(flat)
        # the result is written to `flat` by the kernel itself (in multimem mode: copied out of the staging region
        # before a trailing cross-rank barrier, so a peer's next collective on this workspace cannot overwrite it)
        ops.load_ext(required=True).allreduce_symm(self.peer_ptrs_dev, self.mc_ptr, self.signal_ptrs_dev,
                                                  flat, n, self.rank, self.world, use_multimem)
        return x


class SymmetricFlat:
    """A flat 16-bit buffer in symmetric memory of a (data-parallel) group: same size on every rank, peer-mapped,
    with the NVSwitch multicast mapping when there is one. The data-parallel wrapper and ``FusedAdamW`` keep the flat
    gradient and parameter buffers in it, so that a bucket's reduce-scatter and the parameter all-gather are this
    package's own kernels (``dp_reduce_scatter_kernel`` / ``dp_all_gather_kernel`` in ``csrc/comm.cu``): rank ``r``
    owns elements ``[r * shard, (r + 1) * shard)``."""

    def __init__(self, group, numel: int, dtype: torch.dtype, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.tensor = symm.empty(int(numel), dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.tensor, group)
        self.peer_ptrs_dev = int(self.handle.buffer_ptrs_dev)
        self.signal_ptrs_dev = int(self.handle.signal_pad_ptrs_dev)
        try:
            self.mc_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support else 0
        except Exception:
            self.mc_ptr = 0
        self.tensor.zero_()
        self.shard = -(-int(numel) // (8 * self.world)) * 8      # elements per rank, a multiple of 8
        self.handle.barrier()

    def _mm(self) -> bool:
        return bool(get_config().use_multimem) and self.mc_ptr != 0

    def reduce_scatter_(self, lo: int, hi: int) -> None:
        """Elements [lo, hi) (multiples of 8): this rank's part becomes the sum over the group, in place.
        Collective: every rank of the group calls it with the same range, on a stream of its choice."""
        ops.load_ext(required=True).dp_reduce_scatter(self.tensor, self.peer_ptrs_dev, self.mc_ptr, self.signal_ptrs_dev,
                                                     int(lo), int(hi), self.shard, self.rank, self.world, self._mm())

    def all_gather_(self, lo: int, hi: int) -> None:
        """Elements [lo, hi): every rank's own part is copied into all ranks' buffers. Collective."""
        ops.load_ext(required=True).dp_all_gather(self.tensor, self.peer_ptrs_dev, self.mc_ptr, self.signal_ptrs_dev,
                                                 int(lo), int(hi), self.shard, self.rank, self.world, self._mm())


class CeCombine:
    """Symmetric staging (two halves of 3 x ``cap`` floats) for ``ce_combine_kernel``: the per-row cross-entropy
    statistics of the vocabulary shards are combined over the tensor-parallel group in ONE kernel with one
    cross-rank meeting, instead of a MAX and a SUM all-reduce."""

    CAP = 1 << 16     # rows per call (a chunked LM head hands over a micro-batch's rows at most)

    def __init__(self, group, device) -> None:
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buf = symm.empty(2 * 3 * self.CAP, dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.buf, group)
        self.peer_ptrs_dev = int(self.handle.buffer_ptrs_dev)
        self.signal_ptrs_dev = int(self.handle.signal_pad_ptrs_dev)
        self.counters = torch.zeros(8, dtype=torch.int32, device=device)
        self.buf.zero_()
        self.handle.barrier()

    def __call__(self, mx: torch.Tensor, se: torch.Tensor, tg: torch.Tensor) -> None:
        """In place: every rank ends with the same (max, sum exp relative to it, label logit) per row."""
        ext = ops.load_ext(required=True)
        for s in range(0, mx.numel(), self.CAP):
            e = min(mx.numel(), s + self.CAP)
            ext.ce_combine(mx[s:e], se[s:e], tg[s:e], self.peer_ptrs_dev, self.signal_ptrs_dev, self.counters,
                           self.CAP, self.rank, self.world)


_CE_COMBINERS: Dict[str, CeCombine] = {}


def get_ce_combine(group, device) -> CeCombine:
    name = group.group_name
    c = _CE_COMBINERS.get(name)
    if c is None:
        c = CeCombine(group, device)
        _CE_COMBINERS[name] = c
    return c


def symmetric_flat_usable(group, dtype: torch.dtype, device) -> bool:
    """The data-parallel buffers go to symmetric memory on CUDA devices, over NCCL groups of more than one rank,
    for 16-bit gradients / parameters, when the kernels are built, ``OSLO_B200_DP_SYMMETRIC`` is not switched off and
    the whole group sits on one host. Every condition is the same on all ranks of the group."""
    if group is None or not get_config().dp_symmetric:
        return False
    if torch.device(device).type != "cuda" or dtype not in (torch.bfloat16, torch.float16):
        return False
    if dist.get_backend(group) != "nccl" or dist.get_world_size(group) < 2 or dist.get_world_size(group) > 16:
        return False
    return ops.kernels_available() and group_on_one_node(group)


class _VocabEmbed(torch.autograd.Function):
    """Lookup in a vocabulary-sharded table + its collective as one kernel (``vocab_embed_kernel``): the rank that
    owns a token's row stores it into every rank's staging buffer. Backward is local: every rank holds the whole
    output gradient and scatters the rows of the ids it owns into its shard."""

    @staticmethod
    def forward(ctx, ids, weight, lo, hi, ws):
        flat = ids.reshape(-1).contiguous()
        use_mm = bool(get_config().use_multimem) and ws.has_multicast
        out = ops.load_ext(required=True).vocab_embed(flat, weight, lo, hi, ws.peer_ptrs_dev, ws.mc_ptr, ws.signal_ptrs_dev,
                                                     ws.embed_counters, ws.embed_half, ws.rank, ws.world, use_mm)
        ctx.save_for_backward(flat)
        ctx.cfg = (lo, hi, weight.size(0))
        return out.view(*ids.shape, weight.size(1))

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        lo, hi, rows = ctx.cfg
        owned = (flat >= lo) & (flat < hi)
        local = (flat - lo).masked_fill(~owned, 0)
        g = dy.reshape(flat.numel(), -1).masked_fill(~owned.unsqueeze(-1), 0.0)
        dw = torch.ops.aten.embedding_dense_backward(g, local, rows, -1, False)
        return None, dw, None, None, None


def vocab_embed_usable(ws: "SymmetricWorkspace", ids: torch.Tensor, weight: torch.Tensor) -> bool:
    """16-bit contiguous shard with rows of a multiple of 8 elements, and an output that fits one staging half."""
    return (weight.is_cuda and weight.dtype in (torch.bfloat16, torch.float16) and weight.dim() == 2
            and weight.size(1) % 8 == 0 and weight.is_contiguous()
            and 0 < ids.numel() * weight.size(1) * 2 <= ws.embed_half)


def vocab_embed(ws: "SymmetricWorkspace", ids: torch.Tensor, weight: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    return _VocabEmbed.apply(ids, weight, int(lo), int(hi), ws)


def get_workspace(group, nbytes: Optional[int] = None) -> SymmetricWorkspace:
    """One workspace per process group (created collectively on first use)."""
    name = group.group_name
    ws = _WORKSPACES.get(name)
    want = nbytes or get_config().symm_buffer_mb * 2 ** 20
    if ws is None or ws.numel * 2 < want:
        ws = SymmetricWorkspace(group, want)
        _WORKSPACES[name] = ws
    return ws
