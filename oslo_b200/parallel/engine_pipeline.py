"""Pipeline-parallel engine: contiguous stage partition and a true 1F1B micro-batch schedule
behind the generator API of the reference.

User contract (reference: oslo/parallelism/engine_pipeline.py:262-303, :597-738): ``model(**batch)``
takes keyword arguments only and returns a generator with one output per micro-batch, the same
count on every stage; ``output.loss.backward()`` (or any wrapper that ends in autograd, such as a
grad scaler) must be called inside the loop.

What differs from the reference: its schedule runs one micro-batch through all stages, ring-sends the
full output (logits included) back to every stage, and only then starts the next one, so stages
never overlap. Here stage ``s`` runs ``P-1-s`` forwards ahead before yielding, then alternates one
forward with the backward the user triggers (1F1B). Only the ``[mb, S, H]`` activation and its
gradient cross stage boundaries (every stage slices the batch itself; shapes are known to both
sides so no metadata is exchanged); activations and gradients travel on two separate process
groups so the opposite directions never queue behind each other. Non-last stages yield a proxy
loss: an autograd node whose backward receives the gradient (and the loss value) from the next
stage, so plain autograd drives the whole chain.
"""
from __future__ import annotations

import logging
import os
import pickle
from typing import Any, Callable, Dict, Iterator, List, NamedTuple, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .mpu import MPU

logger = logging.getLogger(__name__)


def one_f_one_b_order(num_stages: int, stage: int, num_micro: int) -> List[str]:
    """The sequence of ``F<i>`` / ``B<i>`` actions stage ``stage`` executes in one step (pure function)."""
    warm = min(num_stages - 1 - stage, num_micro)
    order = [f"F{i}" for i in range(warm)]
    done = warm
    for i in range(num_micro):
        if done < num_micro:
            order.append(f"F{done}")
            done += 1
        order.append(f"B{i}")
    return order


def balanced_partition(num_blocks: int, num_stages: int, head_blocks: float = 1.5, embed_blocks: float = 0.15) -> List[int]:
    """Blocks per stage that minimise the load of the busiest stage when the first stage also embeds the tokens
    (``embed_blocks`` block-equivalents of work) and the last stage also runs the LM head and the loss
    (``head_blocks``). A 1F1B step lasts about (micro-batches + stages - 1) times the busiest stage's time per
    micro-batch, so that stage is what the split should relieve. GPT-J-6B on 4 stages: [7, 7, 8, 6] instead of
    [7, 7, 7, 7] (measured: LM head + loss weigh 1.5 blocks, the embedding 0.15). Among equally good splits the one
    closest to the even split wins; every stage keeps at least one block."""
    L, P = int(num_blocks), int(num_stages)
    if P < 1 or L < P:
        raise ValueError(f"{L} blocks cannot be split over {P} pipeline stages")
    if P == 1:
        return [L]
    best, best_key = None, None
    even = L / P

    def rec(stage: int, left: int, acc: List[int], worst: float) -> None:
        nonlocal best, best_key
        if best_key is not None and worst > best_key[0] + 1e-9:
            return                                    # some stage of this prefix is already busier than the best split
        if stage == P - 1:
            parts = acc + [left]
            worst = max(worst, left + head_blocks)
            key = (round(worst, 6), round(sum((n - even) ** 2 for n in parts), 6), parts)
            if best_key is None or key < best_key:
                best, best_key = parts, key
            return
        lo = max(1, int(even) - 2)
        hi = min(left - (P - 1 - stage), int(even) + 3)
        for n in range(lo, hi + 1):
            rec(stage + 1, left - n, acc + [n], max(worst, n + (embed_blocks if stage == 0 else 0.0)))

    rec(0, L, [], 0.0)
    if best is None or min(best) < 1:      # the window around the even split found nothing valid (tiny models)
        base = L // P
        best = [base] * (P - 1) + [L - base * (P - 1)]
    return best


class MicroLossTensor(torch.Tensor):
    """Marker subclass for the loss yielded on stages that do not own the model head.

    Its value is filled in when the gradient message of that micro-batch arrives; ``backward``
    is ordinary autograd (the proxy node does the receive).
    """

    @staticmethod
    def wrap(t: Tensor) -> "MicroLossTensor":
        return t.as_subclass(MicroLossTensor)


class _ProxyLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, stage_out: Tensor, engine: "PipelineParallelEngine", mb: int):
        ctx.engine, ctx.mb = engine, mb
        ctx.shape, ctx.dtype = stage_out.shape, stage_out.dtype
        return stage_out.new_zeros((), dtype=torch.float32)

    @staticmethod
    def backward(ctx, _g):
        eng: PipelineParallelEngine = ctx.engine
        grad = eng._recv_grad(ctx.mb, ctx.shape, ctx.dtype)
        return grad, None, None


class _TensorSlot(NamedTuple):
    """Stand-in for a tensor inside the pickled structure of a message."""
    index: int
    shape: tuple
    dtype: torch.dtype
    requires_grad: bool


def _strip_tensors(value: Any, tensors: List[Tensor]) -> Any:
    """``value`` with every tensor replaced by a slot; the tensors are appended to ``tensors`` in slot order."""
    if torch.is_tensor(value):
        tensors.append(value)
        return _TensorSlot(len(tensors) - 1, tuple(value.shape), value.dtype, bool(value.requires_grad))
    if isinstance(value, dict):
        items = [(k, _strip_tensors(v, tensors)) for k, v in value.items()]
        try:
            out = type(value)()
            for k, v in items:
                out[k] = v
            return out
        except Exception:      # a mapping class with a constructor of its own: ship it as a plain dict
            return dict(items)
    if isinstance(value, torch.Size):
        return value
    if isinstance(value, (list, tuple, set, frozenset)):
        items = [_strip_tensors(v, tensors) for v in value]
        if isinstance(value, tuple) and hasattr(value, "_fields"):
            return type(value)(*items)
        return type(value)(items)
    return value


def _collect_slots(value: Any, slots: List[_TensorSlot]) -> None:
    if isinstance(value, _TensorSlot):
        slots.append(value)
    elif isinstance(value, dict):
        for v in value.values():
            _collect_slots(v, slots)
    elif isinstance(value, (list, tuple, set, frozenset)) and not isinstance(value, torch.Size):
        for v in value:
            _collect_slots(v, slots)


def _fill_slots(value: Any, received: Dict[int, Tensor]) -> Any:
    if isinstance(value, _TensorSlot):
        return received[value.index]
    if isinstance(value, dict):
        for k in list(value.keys()):
            value[k] = _fill_slots(value[k], received)
        return value
    if isinstance(value, torch.Size):
        return value
    if isinstance(value, (list, tuple, set, frozenset)):
        items = [_fill_slots(v, received) for v in value]
        if isinstance(value, tuple) and hasattr(value, "_fields"):
            return type(value)(*items)
        return type(value)(items)
    return value


class P2PCommunicator:
    """Fixed-shape tensor exchange between neighbouring stages.

    The reference ships whole Python dicts element by element with a type-tagged protocol
    (oslo/parallelism/engine_pipeline.py:741-1199); here both sides derive shape and dtype
    from their own copy of the batch, so a message is exactly one tensor (or one batched pair).

    Every (neighbour pair, direction) is its own two-rank process group, i.e. its own NCCL communicator and
    stream: a channel is a FIFO between exactly two ranks, so a receive that was posted early and still waits for
    its sender can never sit in front of a send to the other neighbour (on one shared communicator all
    point-to-point kernels of a rank run in issue order, and a middle stage that pre-posts "receive activation
    j + 1" before "send activation j" would wait for itself around the ring of 1F1B dependencies). Receives are
    issued from a side stream, so they are ordered after nothing on the compute stream and can land while the
    stage computes; the consumer makes the compute stream wait for exactly the message it needs.
    """

    def __init__(self, mpu: MPU) -> None:
        self.mpu = mpu
        ranks = mpu.get_pipeline_parallel_global_ranks()
        stage = mpu.get_pipeline_parallel_rank()
        self._chan: Dict[tuple, Any] = {}     # (lower stage, "fwd" | "bwd") -> two-rank group
        # every rank creates every group (collective call), in the same order
        for rs in mpu.get_pipeline_parallel_global_ranks_across_all_groups():
            for s in range(len(rs) - 1):
                for direction in ("fwd", "bwd"):
                    g = dist.new_group(ranks=[rs[s], rs[s + 1]], backend=mpu.backend)
                    if rs == ranks and stage in (s, s + 1):
                        self._chan[(s, direction)] = g
        self.side = torch.cuda.Stream() if (mpu.backend == "nccl" and torch.cuda.is_available()) else None
        mpu._p2p_communicator = self         # what MPU.get_p2p_communication_groups() / MPU.p2p() look up

    def _rank(self, stage: int) -> int:
        return self.mpu.stage_to_global_rank(stage)

    def _post(self, ops):
        if len(ops) == 1:
            op = ops[0]
            return [op.op(op.tensor, op.peer, group=op.group)]
        return dist.batch_isend_irecv(ops)       # one NCCL group launch for the whole message

    def send(self, tensors: List[Tensor], dst_stage: int, direction: Optional[str] = None) -> List[Any]:
        """Send ``tensors`` as one message to a neighbouring stage; returns the work handles. Without ``direction``
        this is the reference's ``send(value, recv_stage)``: any value, blocking (``send_object``)."""
        if direction is None:
            self.send_object(tensors, dst_stage)
            return []
        me = self.mpu.get_pipeline_parallel_rank()
        g = self._chan[(min(me, dst_stage), direction)]
        ops = [dist.P2POp(dist.isend, t.contiguous(), self._rank(dst_stage), group=g) for t in tensors]
        return self._post(ops)

    def recv(self, tensors, src_stage: Optional[int] = None, direction: Optional[str] = None):
        """Post the receive of one message (same tensor count and shapes as the sender's). With a single argument
        this is the reference's ``recv(send_stage)``: returns the value the neighbour sent (``recv_object``)."""
        if direction is None:
            return self.recv_object(tensors if src_stage is None else src_stage)
        me = self.mpu.get_pipeline_parallel_rank()
        g = self._chan[(min(me, src_stage), direction)]
        ops = [dist.P2POp(dist.irecv, t, self._rank(src_stage), group=g) for t in tensors]
        if self.side is None:
            return self._post(ops)
        with torch.cuda.stream(self.side):
            return self._post(ops)

    # ------------------------------------------------------------------ arbitrary values (cold path)
    # The reference's communicator moves any Python value between stages - bool, int, float, complex, str, type,
    # None, list, tuple, set, dict, torch.Size, tensors, nested - one small broadcast per scalar and per container
    # element (oslo/parallelism/engine_pipeline.py:823-1199). The same capability here is three kinds of message per
    # value: a two-number header, the pickled structure with every tensor replaced by a (shape, dtype) slot, and the
    # tensors themselves, device to device. Not used by the training schedule, which only ever sends activations.
    def send_object(self, value: Any, dst_stage: int) -> None:
        """Send ``value`` (any picklable structure; tensors at any depth travel as tensors) to a neighbouring stage."""
        me = self.mpu.get_pipeline_parallel_rank()
        if abs(dst_stage - me) != 1:
            raise ValueError(f"stage {me} can only send to a neighbouring stage, not to {dst_stage}")
        g = self._chan[(min(me, dst_stage), "fwd" if dst_stage > me else "bwd")]
        dst = self._rank(dst_stage)
        tensors: List[Tensor] = []
        payload = pickle.dumps(_strip_tensors(value, tensors), protocol=pickle.HIGHEST_PROTOCOL)
        dev = self.mpu.device
        dist.send(torch.tensor([len(payload), len(tensors)], dtype=torch.int64, device=dev), dst, group=g)
        dist.send(torch.frombuffer(bytearray(payload), dtype=torch.uint8).to(dev), dst, group=g)
        for t in tensors:
            dist.send(t.detach().to(dev).contiguous(), dst, group=g)

    def recv_object(self, src_stage: int) -> Any:
        """Receive what the neighbouring stage ``src_stage`` passed to ``send_object``; tensors arrive on this rank's
        device with the sender's ``requires_grad`` flag."""
        me = self.mpu.get_pipeline_parallel_rank()
        if abs(src_stage - me) != 1:
            raise ValueError(f"stage {me} can only receive from a neighbouring stage, not from {src_stage}")
        g = self._chan[(min(me, src_stage), "fwd" if src_stage < me else "bwd")]
        src = self._rank(src_stage)
        dev = self.mpu.device
        head = torch.zeros(2, dtype=torch.int64, device=dev)
        dist.recv(head, src, group=g)
        nbytes, ntensors = (int(v) for v in head.tolist())
        raw = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        dist.recv(raw, src, group=g)
        skeleton = pickle.loads(raw.cpu().numpy().tobytes())
        slots: List[_TensorSlot] = []
        _collect_slots(skeleton, slots)
        if len(slots) != ntensors:
            raise RuntimeError(f"message announces {ntensors} tensors, its structure holds {len(slots)}")
        received = {}
        for slot in sorted(slots, key=lambda x: x.index):
            t = torch.empty(slot.shape, dtype=slot.dtype, device=dev)
            dist.recv(t, src, group=g)
            received[slot.index] = t.requires_grad_(True) if slot.requires_grad else t
        return _fill_slots(skeleton, received)

    def ring_exchange_forward(self, value: Any) -> Any:
        """The first stage's ``value`` travels 0 -> 1 -> ... -> last; every stage returns it
        (reference: oslo/parallelism/engine_pipeline.py:795-807)."""
        stage = self.mpu.get_pipeline_parallel_rank()
        if not self.mpu.is_pipeline_first_stage():
            value = self.recv_object(stage - 1)
        if not self.mpu.is_pipeline_last_stage():
            self.send_object(value, stage + 1)
        return value

    def ring_exchange_backward(self, value: Any) -> Any:
        """The last stage's ``value`` travels last -> ... -> 1 -> 0; every stage returns it (reference: :809-821)."""
        stage = self.mpu.get_pipeline_parallel_rank()
        if not self.mpu.is_pipeline_last_stage():
            value = self.recv_object(stage + 1)
        if not self.mpu.is_pipeline_first_stage():
            self.send_object(value, stage - 1)
        return value

    def alloc(self, shape, dtype, device) -> Tensor:
        """Receive buffer; allocated on the side stream that the receive runs on."""
        if self.side is None:
            return torch.empty(shape, dtype=dtype, device=device)
        with torch.cuda.stream(self.side):
            return torch.empty(shape, dtype=dtype, device=device)

    def finish(self, works: List[Any], tensors: List[Tensor]) -> None:
        """Make the current (compute) stream wait for a posted receive and hand its buffers over to that stream."""
        for w in works:
            w.wait()
        if self.side is not None:
            cur = torch.cuda.current_stream()
            for t in tensors:
                t.record_stream(cur)


def _add_typed_messages() -> None:
    """``send_<kind>(value, recv_stage, send_type=False)`` / ``recv_<kind>(send_stage)`` for the value kinds the
    reference's communicator names one by one (oslo/parallelism/engine_pipeline.py:837-1199). Every message here is
    self-describing, so ``send_type`` is accepted and ignored; both ends check the kind."""
    kinds = {"bool": bool, "int": int, "float": float, "complex": complex, "str": str, "type": type, "none": type(None),
             "list": list, "tuple": tuple, "set": set, "dict": dict, "size": torch.Size, "tensor": Tensor}

    def make(name, kind):
        def send(self, value, recv_stage, send_type=False):
            if not isinstance(value, kind) or (kind is int and isinstance(value, bool)):
                raise TypeError(f"send_{name} got {type(value).__name__}")
            self.send_object(value, recv_stage)

        def recv(self, send_stage):
            value = self.recv_object(send_stage)
            if not isinstance(value, kind):
                raise TypeError(f"recv_{name} got {type(value).__name__} from stage {send_stage}")
            return value

        send.__name__, recv.__name__ = f"send_{name}", f"recv_{name}"
        return send, recv

    for name, kind in kinds.items():
        snd, rcv = make(name, kind)
        setattr(P2PCommunicator, f"send_{name}", snd)
        setattr(P2PCommunicator, f"recv_{name}", rcv)


_add_typed_messages()


class _StageModule(nn.ModuleList):
    """This rank's modules; calling it runs the pipeline generator (what DDP / ZeRO wrappers call)."""

    def forward(self, *args, **kwargs):
        return self._engine_forward(*args, **kwargs)


class PipelineParallelEngine:
    def __init__(self, model: nn.Module, mpu: MPU, micro_batch_size: int = 1, device=None,
                 partition: Optional[List[int]] = None) -> None:
        """``partition``: blocks per stage (e.g. ``[7, 8, 7, 6]``), when the stages should not get the reference's even
        split (floor(L / P) each, remainder to the last stage, oslo/parallelism/mpu.py:934-948): the last stage also
        runs the LM head and the loss, which for GPT-J-6B weigh about as much as one and a half blocks."""
        self.model, self.mpu = model, mpu
        self.partition = [int(n) for n in partition] if partition else None
        self.micro_batch_size = int(micro_batch_size)
        self.device = device or mpu.device
        self.pp = mpu.get_pipeline_parallel_world_size()
        self.stage = mpu.get_pipeline_parallel_rank()
        self.first, self.last = self.stage == 0, self.stage == self.pp - 1
        self._owned_ids: set = set()
        self._owned_params: set = set()
        self._key_stage: Dict[str, int] = {}
        self.block_range = (0, 0)
        self.stage_module: Optional[_StageModule] = None
        self.p2p: Optional[P2PCommunicator] = None
        self._grad_hooks_cb: List[Callable[[], None]] = []
        self.on_last_backward: Optional[Callable[[bool], None]] = None
        # Receives are posted one micro-batch ahead only after this many complete runs of the generator (per mode:
        # training / no-grad). A receive that is posted early is a kernel that spins until its sender runs; during the
        # first pass every kernel is launched for the first time, CUDA loads a kernel's module at its first launch, and
        # that load can wait for all running kernels of the context - the spinning receive among them, whose sender may
        # in turn be waiting (on the host, in NCCL's first-use connection set-up, or on the device) for this rank to get
        # further. Without look-ahead every receive is posted exactly when its data is needed, which is acyclic.
        self.prepost_after = int(os.environ.get("OSLO_B200_PP_PREPOST_AFTER", "1"))
        self._runs = {True: 0, False: 0}
        self.zero_stage: Optional[int] = None  # of a DeepSpeed engine around this model; looked up at the first call
        self.profile = False                  # record CUDA events around every forward / backward (schedule_report)
        self._events: Dict[tuple, Dict[str, Any]] = {}

    # ------------------------------------------------------------------ partition
    def _bounds(self) -> List[int]:
        """Block index at which every stage starts, plus the block count at the end."""
        L = self.model.num_blocks()
        if self.partition is None:
            return self.mpu.make_pipeline_partition(L, self.pp)
        if len(self.partition) != self.pp or sum(self.partition) != L or min(self.partition) < 1:
            raise ValueError(f"pipeline_partition {self.partition} must give {self.pp} stages at least one block each "
                             f"and {L} blocks in total")
        bounds = [0]
        for n in self.partition:
            bounds.append(bounds[-1] + n)
        return bounds

    def _stage_modules(self, stage: int) -> List[nn.Module]:
        model, cfg = self.model, self.model.config
        bounds = self._bounds()
        mods: List[nn.Module] = []
        for policy in model.get_layer_policies():
            blocks = policy.block_layers(model, cfg)
            if stage == 0:
                mods += [l.module for l in policy.word_embedding(model, cfg) + policy.preblock_layers(model, cfg)]
            mods += blocks[bounds[stage]:bounds[stage + 1]]
            if stage == self.pp - 1:
                mods += [l.module for l in policy.postblock_layers(model, cfg)]
        if stage == self.pp - 1:
            mods += [l.module for l in model.get_head_layers() if l.module is not None]
        return mods

    def assign_stages(self) -> None:
        L = self.model.num_blocks()
        if L < self.pp:
            raise ValueError(f"{L} blocks cannot be split over {self.pp} pipeline stages")
        bounds = self._bounds()
        self.block_range = (bounds[self.stage], bounds[self.stage + 1])
        names = {}
        for n, p in self.model.named_parameters(remove_duplicate=False):
            names.setdefault(id(p), []).append(n)
        for n, b in self.model.named_buffers(remove_duplicate=False):
            names.setdefault(id(b), []).append(n)
        for s in range(self.pp):
            for m in self._stage_modules(s):
                for sub in m.modules():
                    if s == self.stage:
                        self._owned_ids.add(id(sub))
                for t in list(m.parameters()) + list(m.buffers()):
                    if s == self.stage:
                        self._owned_params.add(id(t))
                    for n in names.get(id(t), []):
                        self._key_stage.setdefault(n, s)
        self._owned_modules = self._stage_modules(self.stage)
        self._owned_keys = {n for tid in self._owned_params for n in names.get(tid, [])}

    def owns(self, module: nn.Module) -> bool:
        return self.pp == 1 or id(module) in self._owned_ids

    def owns_param(self, t: Tensor) -> bool:
        return self.pp == 1 or id(t) in self._owned_params

    def owns_key(self, key: str) -> bool:
        return self.pp == 1 or key in self._owned_keys

    def finalize(self) -> None:
        model = self.model
        for t in list(model.parameters()) + list(model.buffers()):
            if self.pp == 1 or id(t) in self._owned_params:
                if t.device != self.device:
                    t.data = t.data.to(self.device)
            else:
                t.data = torch.empty(0, dtype=t.dtype, device=self.device)
                if isinstance(t, nn.Parameter):
                    t.requires_grad_(False)
        if self.pp == 1:
            return
        self.p2p = P2PCommunicator(self.mpu)
        if self.mpu.backend == "nccl" and torch.cuda.is_available():
            # transfers between stages are kernels that hold an SM each while they wait for the neighbour: keep the
            # persistent GEMM grids off a few SMs so that such a kernel never pushes GEMM work to the end of a launch
            from .. import ops
            from ..config import get_config
            if ops.kernels_available() and get_config().pp_reserved_sms > 0:
                ops.load_ext().set_reserved_sms(int(get_config().pp_reserved_sms))
        sm = _StageModule(self._owned_modules)
        sm._engine_forward = self.forward
        self.stage_module = sm
        # keep the engine and the stage list out of state_dict / module registration
        object.__setattr__(model, "_pipe_engine", self)
        object.__setattr__(model, "_orig_forward", model.forward)
        object.__setattr__(model, "forward", self.forward)

    # ------------------------------------------------------------------ batch handling
    def set_micro_batch_size(self, micro_batch_size: int) -> None:
        """Sequences per micro-batch from the next call on (``generate()`` sets it to the whole batch)."""
        self.micro_batch_size = int(micro_batch_size)

    def parallelize(self) -> None:
        """Assign the stages and move / drop parameters in one call (what ``parallelize`` /
        ``from_pretrained_with_parallel`` do around the tensor-parallel engine)."""
        self.assign_stages()
        self.finalize()

    @staticmethod
    def guess_batch_size(kwargs: Dict[str, Any]) -> int:
        """Batch size of a call's keyword arguments: the leading dimension of ``input_ids``, ``attention_mask`` or
        ``labels`` (reference: oslo/parallelism/engine_pipeline.py:306-322), else of the first batched tensor
        (``inputs_embeds``, ...)."""
        for key in ("input_ids", "attention_mask", "labels"):
            v = kwargs.get(key)
            if v is not None:
                if not torch.is_tensor(v):
                    raise ValueError(f"``{key}`` must be a tensor of shape (batch_size, ...), got {type(v).__name__}")
                return v.size(0)
        for v in kwargs.values():
            if torch.is_tensor(v) and v.dim() >= 1:
                return v.size(0)
        kinds = {k: type(v).__qualname__ for k, v in kwargs.items()}
        raise ValueError(f"no batched tensor found in the inputs (input_ids, attention_mask, labels, ...): {kinds}")

    def _split_batches(self, kwargs: Dict[str, Any]) -> List[Dict[str, Any]]:
        bsz = self.guess_batch_size(kwargs)
        mbs = max(1, min(self.micro_batch_size, bsz))
        if bsz % mbs:
            raise ValueError(f"batch size {bsz} is not divisible by micro_batch_size {mbs}")
        n = bsz // mbs
        out = [dict() for _ in range(n)]
        for k, v in kwargs.items():
            if torch.is_tensor(v) and v.dim() >= 1 and v.size(0) == bsz:
                for i, c in enumerate(torch.chunk(v, n, dim=0)):
                    out[i][k] = c.to(self.device, non_blocking=True)
            else:
                for i in range(n):
                    out[i][k] = v
        return out

    def _hidden_shape(self, kw: Dict[str, Any]):
        ref = kw.get("input_ids")
        if ref is None:
            ref = kw.get("inputs_embeds")
        b = ref.numel() // ref.size(-1) if kw.get("input_ids") is not None else ref.size(0)
        s = ref.size(-1) if kw.get("input_ids") is not None else ref.size(1)
        cfg = self.model.config
        h = getattr(cfg, "n_embd", None) or cfg.hidden_size
        if getattr(self.model.base_model, "sequence_parallel", False) and self.mpu.tp > 1:
            return (1, b * s // self.mpu.tp, h)
        return (b, s, h)

    # ------------------------------------------------------------------ stage execution
    def _run_stage(self, mb_kw: Dict[str, Any], hidden: Optional[Tensor]) -> Dict[str, Any]:
        model = self.model
        if self.first:
            kw = model.preblock_fn(**mb_kw)
        else:
            # head models that take extra inputs (multiple-choice ids and labels) normalise them themselves
            kw = (getattr(model, "prepare_fn", None) or model.base_model.prepare_fn)(**mb_kw)
            kw["hidden_states"] = hidden
        for i in range(*self.block_range):
            kw = model.block_fn(layer_id=i, **kw)
        if self.last:
            kw = model.postblock_fn(**kw)
            kw = model.head_fn(**kw)
            kw = model.loss_fn(**kw)
        elif kw.get("cache") is not None:
            kw["cache"].advance(kw["_seq"])   # what postblock_fn does on the last stage: this stage's layers are filled
        return kw

    def _post_recv_grad(self, mb: int, shape, dtype) -> None:
        """Post the receive of micro-batch ``mb``'s output gradient (+ loss value) from the next stage."""
        if mb in self._grad_recv:
            return
        g = self.p2p.alloc(shape, dtype, self.device)
        lossv = self.p2p.alloc((1,), torch.float32, self.device)
        self._grad_recv[mb] = (g, lossv, self.p2p.recv([g, lossv], self.stage + 1, "bwd"))

    def _recv_grad(self, mb: int, shape, dtype) -> Tensor:
        self._post_recv_grad(mb, shape, dtype)
        g, lossv, works = self._grad_recv.pop(mb)
        self.p2p.finish(works, [g, lossv])
        proxy = self._proxies.pop(mb, None)
        if proxy is not None:
            proxy.data.copy_(lossv[0])
        self._loss_values[mb] = lossv
        self._mark("B", mb, "start")
        return g

    def _make_input_hook(self, mb: int):
        def hook(grad: Tensor):
            lossv = self._loss_values.pop(mb, None)
            if lossv is None:
                lossv = torch.zeros(1, dtype=torch.float32, device=self.device)
            self._pending += self.p2p.send([grad, lossv], self.stage - 1, "bwd")
            self._mark("B", mb, "end")
            return grad
        return hook

    # ------------------------------------------------------------------ schedule timing (optional)
    def _mark(self, kind: str, mb: int, edge: str) -> None:
        """With ``profile = True``: CUDA events around every forward and backward of this stage."""
        if not self.profile or not torch.cuda.is_available() or self.device.type != "cuda":
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.setdefault((kind, mb), {})[edge] = ev

    def schedule_report(self) -> Dict[str, float]:
        """Busy time of this stage in the last step (sum of its forward / backward spans, device-timed), the span
        from its first to its last event, and the idle share of that span. Call after a synchronize. The ideal
        1F1B idle share with P stages and m micro-batches of equal cost is (P - 1) / (m + P - 1)."""
        done = [e for e in self._events.values() if "start" in e and "end" in e]
        spans = sum(e["start"].elapsed_time(e["end"]) for e in done)
        total = 0.0
        if done:
            first, last = done[0]["start"], done[0]["end"]
            for e in done[1:]:
                if e["start"].elapsed_time(first) > 0:      # e started before the earliest start seen so far
                    first = e["start"]
                if last.elapsed_time(e["end"]) > 0:
                    last = e["end"]
            total = first.elapsed_time(last)
        m = len({mb for (_k, mb) in self._events})
        return {"busy_ms": spans, "span_ms": total, "idle_share": (1.0 - spans / total) if total > 0 else 0.0,
                "ideal_idle_share": (self.pp - 1) / (m + self.pp - 1) if m else 0.0, "micro_batches": m,
                "stage": self.stage}

    def _guess_zero_stage(self) -> int:
        """ZeRO stage of a DeepSpeed engine that is driving this model, found among the local variables of the calling
        frames (reference: oslo/parallelism/engine_pipeline.py:457-480). Stages 2 and 3 partition gradients /
        parameters in ways that do not survive several micro-batch backward passes per step, so they are refused."""
        import inspect
        try:
            from deepspeed.runtime.engine import DeepSpeedEngine as _Engine
        except Exception:      # DeepSpeed is not installed: recognise an engine by its class name
            _Engine = None
        frame = inspect.currentframe()
        try:
            while frame is not None:
                for obj in list(frame.f_locals.values()):
                    is_engine = isinstance(obj, _Engine) if _Engine is not None else type(obj).__name__ == "DeepSpeedEngine"
                    if is_engine and callable(getattr(obj, "zero_optimization", None)):
                        if obj.zero_optimization():
                            return int(obj.zero_optimization_stage())
                        return 0
                frame = frame.f_back
        finally:
            del frame
        return 0

    def forward(self, *args, **kwargs) -> Iterator[Any]:
        if args:
            raise ValueError("pipeline-parallel models take keyword arguments only, e.g. model(**batch)")
        if self.zero_stage is None:
            self.zero_stage = self._guess_zero_stage()
        if self.zero_stage > 1:
            raise RuntimeError("ZeRO-2 and ZeRO-3 are incompatible with pipeline parallelism "
                               "(https://github.com/microsoft/DeepSpeed/issues/1110); use ZeRO stage 0 or 1")
        return self._generator(kwargs)

    def _generator(self, kwargs: Dict[str, Any]) -> Iterator[Any]:
        batches = self._split_batches(kwargs)
        m = len(batches)
        train = torch.is_grad_enabled()
        self._pending: List[Any] = []
        self._proxies: Dict[int, Tensor] = {}
        self._loss_values: Dict[int, Tensor] = {}
        self._grad_recv: Dict[int, Any] = {}
        self._events: Dict[tuple, Dict[str, Any]] = {}
        model = self.model
        dtype = model.dtype
        outputs: Dict[int, Any] = {}
        recv_buf: Dict[int, Any] = {}
        out_shapes: Dict[int, Any] = {}

        lookahead = self._runs[train] >= self.prepost_after

        def post_recv(j: int, ahead: bool = False) -> None:
            if self.first or j >= m or j in recv_buf or (ahead and not lookahead):
                return
            buf = self.p2p.alloc(self._hidden_shape(batches[j]), dtype, self.device)
            recv_buf[j] = (buf, self.p2p.recv([buf], self.stage - 1, "fwd"))

        def do_forward(j: int) -> None:
            hidden = None
            if not self.first:
                post_recv(j)
                hidden, works = recv_buf.pop(j)
                post_recv(j + 1, ahead=True)      # the next activation may arrive while this one is being used
                self.p2p.finish(works, [hidden])
                if train:
                    hidden.requires_grad_(True)
                    hidden.register_hook(self._make_input_hook(j))
            self._mark("F", j, "start")
            kw = self._run_stage(batches[j], hidden)
            self._mark("F", j, "end")
            if not self.last:
                hs = kw["hidden_states"]
                self._pending += self.p2p.send([hs.detach()], self.stage + 1, "fwd")
                if train:
                    out_shapes[j] = (hs.shape, hs.dtype)
                    proxy = MicroLossTensor.wrap(_ProxyLoss.apply(hs, self, j))
                    self._proxies[j] = proxy
                    kw["loss"] = proxy
                kw.setdefault("logits", None)
                kw.setdefault("loss", None)
                outputs[j] = self._organize_partial(kw)
            else:
                if train and kw.get("loss") is not None and not self.first:
                    self._loss_values[j] = kw["loss"].detach().float().reshape(1)
                outputs[j] = model.organize_fn(**kw)

        if not train:
            for j in range(m):
                do_forward(j)
                yield self._broadcast_output(outputs.pop(j))
            self._flush()
            self._runs[False] += 1
            return

        warm = min(self.pp - 1 - self.stage, m)
        done = 0
        if self.on_last_backward is not None and m > 1:
            # a data-parallel wrapper reduces gradients during the LAST micro-batch's backward only; say so before the
            # first one, so that calling the model directly (not through the wrapper's forward) cannot leave the
            # reduction switched on for every micro-batch
            self.on_last_backward(False)
        for _ in range(warm):
            do_forward(done)
            done += 1
        for i in range(m):
            if not self.last and i in out_shapes and lookahead:
                # the gradient of micro-batch i is the next message from the stage below: post its receive before
                # the forward that precedes backward i is enqueued, so it can land during that forward
                self._post_recv_grad(i, *out_shapes.pop(i))
            if done < m:
                do_forward(done)
                done += 1
            if i == m - 1 and self.on_last_backward is not None:
                self.on_last_backward(True)
            if self.last:
                self._mark("B", i, "start")
            yield outputs.pop(i)
            if self.first:
                self._mark("B", i, "end")         # no input hook on the first stage: backward i ends when the user returns
        self._flush()
        self._allreduce_tied_embedding()
        self._runs[True] += 1

    def _organize_partial(self, kw: Dict[str, Any]):
        """Output object of a stage that has no head: same type as the last stage's, loss = proxy."""
        kw = dict(kw)
        for k in ("all_hidden_states", "all_attentions"):
            kw.setdefault(k, None)
        kw.setdefault("return_dict", True)
        try:
            return self.model.organize_fn(**kw)
        except Exception:  # head-specific fields missing on this stage
            from ..modeling_utils import ModelOutput
            return ModelOutput(loss=kw.get("loss"))

    def _flush(self) -> None:
        for w in self._pending:
            w.wait()
        self._pending = []

    # ------------------------------------------------------------------ collectives around the schedule
    def _broadcast_output(self, out):
        """Inference: every stage returns what the last stage computed (tensors only; caches stay local)."""
        group = self.mpu.get_pipeline_parallel_group()
        src = self.mpu.stage_to_global_rank(self.pp - 1)
        if self.last:
            items = [(k, tuple(v.shape), v.dtype) for k, v in out.items() if torch.is_tensor(v)]
            meta = [items, type(out)]
        else:
            meta = [None, None]
        dist.broadcast_object_list(meta, src=src, group=group)
        items, cls = meta
        res = out if self.last else cls()
        for k, shape, dt in items:
            t = out[k].contiguous() if self.last else torch.empty(shape, dtype=dt, device=self.device)
            dist.broadcast(t, src=src, group=group)
            if not self.last:
                res[k] = t
        if not self.last and hasattr(out, "get") and out.get("past_key_values") is not None:
            res["past_key_values"] = out["past_key_values"]
        return res

    def _allreduce_tied_embedding(self) -> None:
        """Sum the gradients of an embedding shared by the first and the last stage
        (reference: oslo/parallelism/engine_pipeline.py:439-451)."""
        model = self.model
        if not (self.first or self.last) or self.pp == 1:
            return
        if not getattr(model.config, "tie_word_embeddings", True) or model.get_output_embeddings() is None:
            return
        w = model.get_input_embeddings().weight
        if w.grad is None:
            w.grad = torch.zeros_like(w)
        dist.all_reduce(w.grad, group=self.mpu.get_embedding_tied_group())


class PipelineDeparallelEngine:
    """Collect every stage's tensors onto all ranks of a pipeline group (cold path, per-tensor broadcast)."""

    def __init__(self, model: nn.Module, mpu: MPU) -> None:
        self.model, self.mpu = model, mpu

    def gather_state(self, state: Dict[str, Tensor]) -> Dict[str, Tensor]:
        pp = self.mpu.get_pipeline_parallel_world_size()
        if pp == 1:
            return dict(state)
        eng: PipelineParallelEngine = self.model._pipe_engine
        group = self.mpu.get_pipeline_parallel_group()
        out: Dict[str, Tensor] = {}
        for key in sorted(state.keys()):
            stage = eng._key_stage.get(key, 0)
            src = self.mpu.stage_to_global_rank(stage)
            mine = self.mpu.get_pipeline_parallel_rank() == stage
            meta = [(tuple(state[key].shape), state[key].dtype) if mine else None]
            dist.broadcast_object_list(meta, src=src, group=group)
            shape, dt = meta[0]
            t = state[key].detach().to(self.mpu.device).contiguous() if mine else \
                torch.empty(shape, dtype=dt, device=self.mpu.device)
            dist.broadcast(t, src=src, group=group)
            out[key] = t
        return out

    def deparallelize(self) -> nn.Module:
        full = self.gather_state(self.model.state_dict())
        named = dict(self.model.named_parameters(remove_duplicate=False))
        named.update(dict(self.model.named_buffers(remove_duplicate=False)))
        for k, t in full.items():
            if k in named:
                named[k].data = t
                if isinstance(named[k], nn.Parameter):
                    named[k].requires_grad_(True)
        if hasattr(self.model, "_orig_forward"):
            object.__setattr__(self.model, "forward", self.model._orig_forward)
        return self.model
