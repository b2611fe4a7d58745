"""Model-parallel unit: process-group topology and autograd-aware collectives.

Rank layout (identical to the reference so that checkpoints and DeepSpeed-style
engines see the same groups; reference: oslo/parallelism/mpu.py:198-351)::

    global_rank = pp_stage * (world / pp) + dp_rank * tp + tp_rank

* tensor-parallel groups are runs of ``tp`` consecutive ranks,
* pipeline-parallel groups stride by ``world / pp``,
* data-parallel groups stride by ``tp`` inside one pipeline stage,
* a model-parallel group is every rank that shares one ``dp_rank``.

Unlike the reference (NCCL hard-coded, oslo/parallelism/mpu.py:191-196) the
backend follows the device: ``nccl`` on CUDA, ``gloo`` on CPU, so every piece of
parallel logic can be exercised by CPU ranks.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor


def _default_backend() -> str:
    forced = os.environ.get("OSLO_B200_BACKEND")
    if forced:
        return forced
    return "nccl" if torch.cuda.is_available() else "gloo"


def ceil_split_sizes(total: int, parts: int) -> List[int]:
    """Sizes produced by ``torch.chunk(total, parts)``: ceil-sized chunks, last one short.

    50257 over 4 -> [12565, 12565, 12565, 12562] (reference: oslo/modeling_utils.py:18-32).
    """
    step = -(-total // parts)
    sizes = []
    left = total
    for _ in range(parts):
        take = max(0, min(step, left))
        sizes.append(take)
        left -= take
    return sizes


class MPU:
    """Topology + collectives for tensor / pipeline / data parallelism."""

    def __init__(
        self,
        tensor_parallel_size: int = 1,
        pipeline_parallel_size: int = 1,
        backend: Optional[str] = None,
        timeout_s: Optional[float] = None,
    ) -> None:
        self.backend = backend or _default_backend()
        self.initialize_distributed(self.backend, timeout_s)
        world = dist.get_world_size()
        rank = dist.get_rank()
        tp, pp = int(tensor_parallel_size), int(pipeline_parallel_size)
        if tp < 1 or pp < 1:
            raise ValueError("parallel sizes must be >= 1")
        if tp * pp > world:
            raise ValueError(f"tp({tp}) * pp({pp}) exceeds world size {world}")
        if world % (tp * pp) != 0:
            raise ValueError(f"world size {world} is not divisible by tp*pp = {tp * pp}")
        self.world_size, self.rank = world, rank
        self.tp, self.pp, self.dp = tp, pp, world // (tp * pp)
        per_stage = world // pp
        self.pp_rank = rank // per_stage
        self.dp_rank = (rank % per_stage) // tp
        self.tp_rank = rank % tp
        self.device = (
            torch.device("cuda", torch.cuda.current_device())
            if self.backend == "nccl"
            else torch.device("cpu")
        )

        # every rank must create every group, in the same order
        self._tp_group = self._dp_group = self._pp_group = self._mp_group = self._emb_group = None
        self._tp_ranks: List[int] = []
        self._pp_ranks: List[int] = []
        self._dp_ranks: List[int] = []
        self._mp_ranks: List[int] = []
        self._emb_ranks: List[int] = []
        self._all_pp_ranks: List[List[int]] = []
        for ranks in self.layout_tensor_groups(world, tp):
            g = self._new_group(ranks)
            if rank in ranks:
                self._tp_group, self._tp_ranks = g, ranks
        for ranks in self.layout_data_groups(world, tp, pp):
            g = self._new_group(ranks)
            if rank in ranks:
                self._dp_group, self._dp_ranks = g, ranks
        for ranks in self.layout_pipeline_groups(world, pp):
            g = self._new_group(ranks)
            self._all_pp_ranks.append(ranks)
            if rank in ranks:
                self._pp_group, self._pp_ranks = g, ranks
        for ranks in self.layout_model_groups(world, tp, pp):
            g = self._new_group(ranks)
            if rank in ranks:
                self._mp_group, self._mp_ranks = g, ranks
        for ranks in self.layout_pipeline_groups(world, pp):
            emb = [ranks[0]] if pp == 1 else [ranks[0], ranks[-1]]
            g = self._new_group(emb)
            if rank in emb:
                self._emb_group, self._emb_ranks = g, emb
        # which host every rank runs on, asked once here (all ranks are present): the paths that map peers' memory
        # (symmetric.group_on_one_node) then know the answer for this MPU's groups without another collective
        from .symmetric import node_identity, remember_group_nodes
        self.node_of_rank: List[str] = [None] * world
        if world > 1:
            dist.all_gather_object(self.node_of_rank, node_identity())
        else:
            self.node_of_rank = [node_identity()]
        for g, ranks in ((self._tp_group, self._tp_ranks), (self._dp_group, self._dp_ranks),
                         (self._pp_group, self._pp_ranks), (self._mp_group, self._mp_ranks)):
            if g is not None:
                remember_group_nodes(g, [self.node_of_rank[r] for r in ranks])

    # ------------------------------------------------------------------ layout (pure)
    @staticmethod
    def layout_tensor_groups(world: int, tp: int) -> List[List[int]]:
        return [list(range(i * tp, (i + 1) * tp)) for i in range(world // tp)]

    @staticmethod
    def layout_pipeline_groups(world: int, pp: int) -> List[List[int]]:
        per_stage = world // pp
        return [list(range(i, world, per_stage)) for i in range(per_stage)]

    @staticmethod
    def layout_data_groups(world: int, tp: int, pp: int) -> List[List[int]]:
        per_stage = world // pp
        out = []
        for s in range(pp):
            lo, hi = s * per_stage, (s + 1) * per_stage
            for j in range(tp):
                out.append(list(range(lo + j, hi, tp)))
        return out

    @staticmethod
    def layout_model_groups(world: int, tp: int, pp: int) -> List[List[int]]:
        per_stage = world // pp
        dp = per_stage // tp
        out = []
        for d in range(dp):
            ranks = []
            for s in range(pp):
                base = s * per_stage + d * tp
                ranks.extend(range(base, base + tp))
            out.append(ranks)
        return out

    # ------------------------------------------------------------------ bootstrap
    @staticmethod
    def initialize_distributed(backend: Optional[str] = None, timeout_s: Optional[float] = None) -> None:
        """Join the default process group from RANK / WORLD_SIZE / MASTER_* (idempotent)."""
        if dist.is_initialized():
            return
        backend = backend or _default_backend()
        rank = int(os.environ.get("RANK", 0))
        world = int(os.environ.get("WORLD_SIZE", 1))
        local_rank = int(os.environ.get("LOCAL_RANK", rank))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs: Dict[str, Any] = {}
        if timeout_s is None and os.environ.get("OSLO_B200_PG_TIMEOUT_S"):
            timeout_s = float(os.environ["OSLO_B200_PG_TIMEOUT_S"])
        if timeout_s is not None:
            kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
        if backend == "nccl":
            torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
            if os.environ.get("OSLO_B200_NCCL_EAGER_INIT", "1") != "0":
                # binds the device now and creates every group's communicator by splitting the world communicator
                # (quick group creation). All point-to-point operations of such a group share the group's one
                # communicator and stream, which is why the pipeline engine gives every (neighbour pair, direction) a
                # group of its own.
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        attempt = os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")
        if attempt != "0":         # (all workers of one attempt see the same count)
            # Workers re-launched by `torchrun --max-restarts` meet through the SAME key-value store as the attempt
            # before them, and a sub-group's rendezvous keys are named after the group ("1/...", "2/..."): without a
            # prefix of their own the new ranks would read the addresses (gloo) or the communicator id (NCCL) that the
            # dead ranks left there.
            from torch.distributed.rendezvous import rendezvous
            it = rendezvous("env://", rank, world, **({"timeout": kwargs["timeout"]} if "timeout" in kwargs else {}))
            store, rank, world = next(it)
            kwargs["store"] = dist.PrefixStore(f"attempt_{attempt}/", store)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)

    def _new_group(self, ranks: Sequence[int]):
        return dist.new_group(ranks=list(ranks), backend=self.backend)

    # ------------------------------------------------------------------ getters (Megatron / DeepSpeed names)
    def model_parallel_is_initialized(self) -> bool:
        return self._tp_group is not None and self._pp_group is not None and self._dp_group is not None

    def get_data_parallel_group(self):
        return self._dp_group

    def get_model_parallel_group(self):
        return self._mp_group

    def get_tensor_parallel_group(self):
        return self._tp_group

    def get_pipeline_parallel_group(self):
        return self._pp_group

    def get_embedding_tied_group(self):
        return self._emb_group

    def get_data_parallel_world_size(self) -> int:
        return self.dp

    def get_model_parallel_world_size(self) -> int:
        return self.tp * self.pp

    def get_tensor_parallel_world_size(self) -> int:
        return self.tp

    def get_pipeline_parallel_world_size(self) -> int:
        return self.pp

    def get_embedding_tied_world_size(self) -> int:
        return len(self._emb_ranks)

    def get_data_parallel_rank(self) -> int:
        return self.dp_rank

    def get_model_parallel_rank(self) -> int:
        return self._mp_ranks.index(self.rank)

    def get_tensor_parallel_rank(self) -> int:
        return self.tp_rank

    def get_pipeline_parallel_rank(self) -> int:
        return self.pp_rank

    def get_tensor_parallel_src_rank(self) -> int:
        return (self.rank // self.tp) * self.tp

    def is_pipeline_first_stage(self) -> bool:
        return self.pp_rank == 0

    def is_pipeline_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    def get_tensor_parallel_global_ranks(self) -> List[int]:
        return list(self._tp_ranks)

    def get_data_parallel_global_ranks(self) -> List[int]:
        return list(self._dp_ranks)

    def get_pipeline_parallel_global_ranks(self) -> List[int]:
        return list(self._pp_ranks)

    def get_pipeline_parallel_global_ranks_across_all_groups(self) -> List[List[int]]:
        return [list(r) for r in self._all_pp_ranks]

    def get_pipeline_model_parallel_global_ranks_per_group(self) -> List[int]:
        return list(self._pp_ranks)

    def get_embedding_global_ranks(self) -> List[int]:
        return list(self._emb_ranks)

    def stage_to_global_rank(self, stage: int) -> int:
        return self._pp_ranks[stage]

    def get_p2p_communication_groups(self):
        """``{(source global rank, destination global rank): two-rank group}`` for the neighbour channels this rank
        takes part in (reference: oslo/parallelism/mpu.py:321-368). The groups belong to the pipeline engine's
        ``P2PCommunicator`` - one per neighbour pair and direction - and exist once a pipeline-parallel model has been
        built on this MPU; before that the dict is empty and ``p2p`` sends over the pipeline group."""
        comm = getattr(self, "_p2p_communicator", None)
        if comm is None:
            return {}
        out = {}
        for (lower, direction), g in comm._chan.items():
            a, b = self._pp_ranks[lower], self._pp_ranks[lower + 1]
            out[(a, b) if direction == "fwd" else (b, a)] = g
        return out

    def p2p(self, tensor: Tensor, src_stage: int, dst_stage: int) -> bool:
        """Move ``tensor`` from pipeline stage ``src_stage`` to the neighbouring stage ``dst_stage`` (in place on the
        receiver). Every rank of a pipeline group may call it with the same arguments; it returns True on the two
        ranks that took part and False elsewhere. The reference emulates the transfer with a broadcast in a two-rank
        group (oslo/parallelism/mpu.py:892-920); here it is a send / receive on that pair's channel."""
        pp = self.get_pipeline_parallel_world_size()
        if not (0 <= src_stage < pp and 0 <= dst_stage < pp) or abs(src_stage - dst_stage) != 1:
            raise ValueError(f"p2p needs two neighbouring pipeline stages, got src={src_stage}, dst={dst_stage}")
        me = self.get_pipeline_parallel_rank()
        if me not in (src_stage, dst_stage):
            return False
        src, dst = self._pp_ranks[src_stage], self._pp_ranks[dst_stage]
        group = self.get_p2p_communication_groups().get((src, dst), self._pp_group)
        if me == src_stage:
            dist.send(tensor.contiguous(), dst, group=group)
        else:
            dist.recv(tensor, src, group=group)
        return True

    def get_p2p_communication_world_size(self) -> int:
        return 2

    def get_p2p_communication_global_ranks(self) -> List[List[int]]:
        r = self._pp_ranks
        return [[r[i], r[(i + 1) % len(r)]] for i in range(len(r))]

    def destroy_model_parallel(self) -> None:
        for g in (self._tp_group, self._dp_group, self._pp_group, self._mp_group, self._emb_group):
            if g is not None:
                try:
                    dist.destroy_process_group(g)
                except Exception:
                    pass
        self._tp_group = self._dp_group = self._pp_group = self._mp_group = self._emb_group = None

    # ------------------------------------------------------------------ raw collectives (TP group)
    def _reduce(self, x: Tensor) -> Tensor:
        if self.tp == 1:
            return x
        x = x.contiguous()
        if self._small_symm_ok(x):
            # latency-bound sizes (decode steps): one-shot all-reduce kernel over symmetric memory; its
            # signal words reset themselves, so the call can sit inside a captured CUDA graph
            from .symmetric import get_workspace
            return get_workspace(self._tp_group).all_reduce_(x)
        dist.all_reduce(x, group=self._tp_group)
        return x

    def _small_symm_ok(self, x: Tensor) -> bool:
        if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or x.numel() % 8 or x.numel() == 0:
            return False
        from ..config import get_config
        cfg = get_config()
        limit = getattr(cfg, "symm_allreduce_max_bytes", 0)
        if not (bool(limit) and x.numel() * 2 <= limit and not torch.is_grad_enabled()):
            return False
        from .symmetric import group_on_one_node
        return group_on_one_node(self._tp_group)

    def _scatter(self, x: Tensor, dim: int = -1) -> Tensor:
        if self.tp == 1:
            return x
        return torch.chunk(x, self.tp, dim=dim)[self.tp_rank].contiguous()

    def _gather(self, x: Tensor, dim: int = -1, full_size: Optional[int] = None) -> Tensor:
        """All-gather along ``dim``. Shards may be uneven (ceil split); ``full_size`` avoids a size exchange."""
        if self.tp == 1:
            return x
        dim = dim % x.dim()
        if full_size is None:
            mine = torch.tensor([x.size(dim)], device=x.device, dtype=torch.int64)
            sizes_t = [torch.zeros_like(mine) for _ in range(self.tp)]
            dist.all_gather(sizes_t, mine, group=self._tp_group)
            sizes = [int(s.item()) for s in sizes_t]
        else:
            sizes = ceil_split_sizes(full_size, self.tp)
        big = max(sizes)
        if x.size(dim) != big:
            pad_shape = list(x.shape)
            pad_shape[dim] = big - x.size(dim)
            x = torch.cat([x, x.new_zeros(pad_shape)], dim=dim)
        x = x.contiguous()
        parts = [torch.empty_like(x) for _ in range(self.tp)]
        dist.all_gather(parts, x, group=self._tp_group)
        parts = [p.narrow(dim, 0, s) for p, s in zip(parts, sizes)]
        return torch.cat(parts, dim=dim)

    def _reduce_scatter(self, x: Tensor, dim: int = 0) -> Tensor:
        """Sum over the TP group and keep this rank's even chunk along ``dim``."""
        if self.tp == 1:
            return x
        dim = dim % x.dim()
        if x.size(dim) % self.tp:
            raise ValueError(f"dim {dim} of size {x.size(dim)} is not divisible by tp={self.tp}")
        chunks = [c.contiguous() for c in torch.chunk(x, self.tp, dim=dim)]
        out = torch.empty_like(chunks[0])
        if self.backend == "gloo":  # gloo has no reduce_scatter
            full = x.contiguous()
            dist.all_reduce(full, group=self._tp_group)
            return torch.chunk(full, self.tp, dim=dim)[self.tp_rank].contiguous()
        dist.reduce_scatter(out, chunks, group=self._tp_group)
        return out

    # ------------------------------------------------------------------ autograd-aware collectives
    def broadcast(self, x: Tensor) -> Tensor:
        """Identity forward, all-reduce backward (entry of a column-parallel layer)."""
        if self.tp == 1 or not _wants_grad(x):
            return x
        return _Copy.apply(x, self)

    def reduce(self, x: Tensor) -> Tensor:
        """All-reduce forward, identity backward (exit of a row-parallel layer)."""
        if self.tp == 1:
            return x
        if not _wants_grad(x):
            return self._reduce(x)
        return _Reduce.apply(x, self)

    def scatter(self, x: Tensor, dim: int = -1) -> Tensor:
        """Keep this rank's chunk forward, all-gather backward."""
        if self.tp == 1:
            return x
        if not _wants_grad(x):
            return self._scatter(x, dim)
        return _Scatter.apply(x, self, dim)

    def gather(self, x: Tensor, dim: int = -1, full_size: Optional[int] = None) -> Tensor:
        """All-gather forward, keep-own-chunk backward."""
        if self.tp == 1:
            return x
        if not _wants_grad(x):
            return self._gather(x, dim, full_size)
        return _Gather.apply(x, self, dim, full_size)

    def gather_sequence(self, x: Tensor, dim: int = 0) -> Tensor:
        """Sequence-parallel entry: all-gather forward, reduce-scatter backward."""
        if self.tp == 1:
            return x
        if not _wants_grad(x):
            return self._gather(x, dim, x.size(dim) * self.tp)
        return _GatherSeq.apply(x, self, dim)

    def reduce_scatter_sequence(self, x: Tensor, dim: int = 0) -> Tensor:
        """Sequence-parallel exit: reduce-scatter forward, all-gather backward."""
        if self.tp == 1:
            return x
        if not _wants_grad(x):
            return self._reduce_scatter(x, dim)
        return _ReduceScatterSeq.apply(x, self, dim)

    # ------------------------------------------------------------------ pipeline helpers
    def p2p_send(self, tensor: Tensor, dst_stage: int):
        return dist.isend(tensor.contiguous(), dst=self.stage_to_global_rank(dst_stage))

    def p2p_recv(self, tensor: Tensor, src_stage: int):
        return dist.irecv(tensor, src=self.stage_to_global_rank(src_stage))

    @staticmethod
    def make_pipeline_partition(num_items: int, num_parts: int) -> List[int]:
        """Boundaries of a contiguous split: floor(L/P) per stage, remainder to the last stage.

        Reference: oslo/parallelism/mpu.py:934-948.
        """
        base = num_items // num_parts
        bounds = [i * base for i in range(num_parts)] + [num_items]
        return bounds

    @staticmethod
    def extend_pipeline_partition(partition: Sequence[int]) -> List[int]:
        """Stage index of every item, e.g. [0, 2, 5] -> [0, 0, 1, 1, 1]."""
        out: List[int] = []
        for s in range(len(partition) - 1):
            out.extend([s] * (partition[s + 1] - partition[s]))
        return out


def _wants_grad(x: Tensor) -> bool:
    return torch.is_grad_enabled() and x.requires_grad


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mpu):
        ctx.mpu = mpu
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.mpu._reduce(g.clone()), None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mpu):
        return mpu._reduce(x.clone())

    @staticmethod
    def backward(ctx, g):
        return g, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mpu, dim):
        ctx.mpu, ctx.dim, ctx.full = mpu, dim, x.size(dim)
        return mpu._scatter(x, dim)

    @staticmethod
    def backward(ctx, g):
        return ctx.mpu._gather(g, ctx.dim, ctx.full), None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mpu, dim, full_size):
        ctx.mpu, ctx.dim = mpu, dim
        ctx.local = x.size(dim)
        out = mpu._gather(x, dim, full_size)
        sizes = ceil_split_sizes(out.size(dim), mpu.tp)
        ctx.offset = sum(sizes[: mpu.tp_rank])
        return out

    @staticmethod
    def backward(ctx, g):
        return g.narrow(ctx.dim, ctx.offset, ctx.local).contiguous(), None, None, None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mpu, dim):
        ctx.mpu, ctx.dim = mpu, dim
        return mpu._gather(x, dim, x.size(dim) * mpu.tp)

    @staticmethod
    def backward(ctx, g):
        return ctx.mpu._reduce_scatter(g, ctx.dim), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mpu, dim):
        ctx.mpu, ctx.dim = mpu, dim
        return mpu._reduce_scatter(x, dim)

    @staticmethod
    def backward(ctx, g):
        return ctx.mpu._gather(g, ctx.dim, g.size(ctx.dim) * ctx.mpu.tp), None, None


# ---------------------------------------------------------------------- layer policy
@dataclass
class Layer:
    """One parallelisable parameter group of a model (reference: oslo/parallelism/mpu.py:963-976).

    ``weight``/``bias`` are the live parameters, ``module`` the owner whose class is swapped
    according to ``replace``. ``n_fused`` > 1 marks a fused projection such as GPT-2's
    ``c_attn`` (q, k, v stacked along the output dim); ``reversed`` marks the ``[in, out]``
    Conv1D weight layout.
    """

    module: Optional[torch.nn.Module] = None
    weight: Optional[Tensor] = None
    bias: Optional[Tensor] = None
    replace: Optional[dict] = None
    n_fused: int = 1
    reversed: bool = False
    parallel: bool = True
    input_is_parallel: bool = True
    gather_output: bool = False
    tied_embedding: Optional[torch.nn.Module] = None


class LayerPolicy:
    """Static description of where a model family keeps its parallelisable layers.

    Reference: oslo/parallelism/mpu.py:979-1043. Every hook returns a list of ``Layer``.
    """

    @staticmethod
    def reduce_arguments(layer, world_size, config):
        pass

    @staticmethod
    def fused_modules() -> dict:
        return {}

    @staticmethod
    def attn_qkv(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def attn_out(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def attn_norm(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def mlp_in(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def mlp_out(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def mlp_norm(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def word_embedding(model, config) -> List[Layer]:
        return []

    @staticmethod
    def preblock_layers(model, config) -> List[Layer]:
        return []

    @staticmethod
    def block_layers(model, config) -> List[torch.nn.Module]:
        return []

    @staticmethod
    def postblock_layers(model, config) -> List[Layer]:
        return []

    @staticmethod
    def copy_to_all(layer, config) -> List[Layer]:
        return []

    @staticmethod
    def original_layer_class():
        return None
