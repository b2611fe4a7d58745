"""Deployment launcher: serve a tensor/pipeline-parallel model from ONE ordinary Python process.

``Model.from_pretrained_with_parallel(..., deployment=True)`` is called from a plain ``python script.py``
(no launcher). The parent spawns ``tp * pp`` worker processes, each of which joins a process group,
parallelises its copy of the model on its own device and then serves requests; in the parent,
``model.generate`` / ``model.forward`` / ``model(...)`` are proxies that fan the call out to every worker
and return rank 0's result, ``model.fuse()`` switches every worker's copy to the fused kernels, and ``model.cpu()`` /
``.cuda()`` / ``.to()`` shut the workers down (reference: oslo/parallelism/engine_deployment.py:22-375).

Differences from the reference: every wait in the parent has a deadline and checks worker liveness, so a
dead worker raises ``DeploymentError`` instead of hanging; exceptions inside a worker travel back with
their traceback; the same seed is chosen in the parent and handed to all workers (the reference
broadcasts ``time()`` from rank 0); results are rebuilt from ``ModelOutput``'s own pickling, no ``dacite``.
"""
from __future__ import annotations

import os
import queue
import socket
import time
import traceback
from typing import Any, Dict, List, Optional

import torch
import torch.multiprocessing as mp


class DeploymentError(RuntimeError):
    pass


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _to_device(obj, device):
    if torch.is_tensor(obj):
        return obj.to(device)
    if isinstance(obj, dict):
        return _rebuild_mapping(obj, device)
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_device(v, device) for v in obj)
    return obj


def _rebuild_mapping(obj, device):
    out = type(obj)()
    for k, v in obj.items():
        out[k] = _to_device(v, device)
    return out


def _strip_for_pickle(obj):
    """Drop device-resident caches from outputs and move tensors to the host."""
    from ..models.common import StaticKVCache
    if isinstance(obj, StaticKVCache):
        return None
    if torch.is_tensor(obj):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        out = type(obj)()
        for k, v in obj.items():
            out[k] = _strip_for_pickle(v)
        return out
    if isinstance(obj, (list, tuple)):
        return type(obj)(_strip_for_pickle(v) for v in obj)
    return obj


def _worker(rank: int, world: int, port: int, model, par: Dict[str, Any], split_path: Optional[str], in_q, out_q,
            ready, backend: Optional[str], factory=None) -> None:
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port))
        if backend:
            os.environ["OSLO_B200_BACKEND"] = backend
        on_gpu = torch.cuda.is_available() and backend != "gloo"
        if on_gpu:
            torch.cuda.set_device(rank % torch.cuda.device_count())
        if factory is not None:
            # random-init model from its config, built by the worker itself on its own device: nothing of the size
            # of the model crosses the process boundary. The shared seed makes every worker draw the same weights.
            from ..parallelism_utils import set_seed
            cls, config, torch_dtype = factory
            set_seed(par.get("seed"))
            with torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu"):
                model = cls._from_config(config, torch_dtype=torch_dtype)
        model._exec_both_engines(**par)
        if split_path is not None:
            model._load_split_checkpoint_files(split_path)
        model.eval()
        device = model.mpu.device
        ready.set()
        while True:
            msg = in_q.get()
            if msg is None:
                break
            fn, args, kwargs = msg
            try:
                args, kwargs = _to_device(args, device), _to_device(kwargs, device)
                if model.is_pipeline_parallelized() and fn != "generate":
                    ref = next((a for a in list(args) + list(kwargs.values()) if torch.is_tensor(a)), None)
                    if ref is not None:
                        model.set_micro_batch_size(ref.size(0))
                with torch.no_grad():
                    out = getattr(model, fn)(*args, **kwargs)
                    if model.is_pipeline_parallelized() and fn != "generate" and hasattr(out, "__next__"):
                        out = [o for o in out][0]
                    if isinstance(out, torch.nn.Module):     # fuse() returns the model: the parent keeps its own handle
                        out = None
                out_q.put(("ok", _strip_for_pickle(out)))
            except BaseException:  # noqa: BLE001 - reported to the parent
                out_q.put(("error", traceback.format_exc()))
    except BaseException:  # noqa: BLE001
        out_q.put(("fatal", traceback.format_exc()))
        ready.set()
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


class DeploymentParallelEngine:
    def __init__(self, model, tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                 micro_batch_size: int = 1, resize_token_embeddings: Optional[int] = None, seed: Optional[int] = None,
                 sequence_parallel: bool = False, split_checkpoint_path: Optional[str] = None,
                 backend: Optional[str] = None, startup_timeout_s: float = 600.0, request_timeout_s: float = 600.0,
                 factory=None, pipeline_partition: Optional[List[int]] = None, **_unused: Any) -> None:
        """``factory = (model class, config, torch_dtype)``: the workers build the (random-init) model themselves and
        ``model`` is only the parent's handle (its tensors may live on the meta device)."""
        self.model = model
        self.factory = factory
        self.world = int(tensor_parallel_size) * int(pipeline_parallel_size)
        self.par = dict(tensor_parallel_size=tensor_parallel_size, pipeline_parallel_size=pipeline_parallel_size,
                        micro_batch_size=micro_batch_size, resize_token_embeddings=resize_token_embeddings,
                        seed=seed if seed is not None else int(time.time()) % (2 ** 31),
                        sequence_parallel=sequence_parallel, pipeline_partition=pipeline_partition)
        self.split_path = split_checkpoint_path
        self.backend = backend or os.environ.get("OSLO_B200_BACKEND")
        self.startup_timeout_s, self.request_timeout_s = startup_timeout_s, request_timeout_s
        self.procs: List[mp.Process] = []
        self.in_qs, self.out_qs = [], []
        os.environ.setdefault("MKL_SERVICE_FORCE_INTEL", "1")

    # ------------------------------------------------------------------ lifecycle
    def parallelize(self):
        ctx = mp.get_context("spawn")
        port = _free_port()
        readies = []
        for rank in range(self.world):
            in_q, out_q, ready = ctx.Queue(), ctx.Queue(), ctx.Event()
            p = ctx.Process(target=_worker, daemon=True,
                            args=(rank, self.world, port, None if self.factory is not None else self.model, self.par,
                                  self.split_path, in_q, out_q, ready, self.backend, self.factory))
            p.start()
            self.procs.append(p)
            self.in_qs.append(in_q)
            self.out_qs.append(out_q)
            readies.append(ready)
        deadline = time.time() + self.startup_timeout_s
        for rank, ev in enumerate(readies):
            while not ev.wait(0.2):
                self._check_alive("start-up")
                if time.time() > deadline:
                    self.deparallelize()
                    raise DeploymentError(f"worker {rank} did not become ready within {self.startup_timeout_s}s")
        for rank, q in enumerate(self.out_qs):  # a worker that failed during start-up left a message
            try:
                kind, payload = q.get_nowait()
            except queue.Empty:
                continue
            self.deparallelize()
            raise DeploymentError(f"worker {rank} failed during start-up:\n{payload}")
        model = self.model
        object.__setattr__(model, "_deployment_engine", self)
        for fn in ("generate", "forward", "fuse"):
            object.__setattr__(model, fn, _Proxy(self, fn))
        for fn in ("cpu", "cuda", "to"):
            object.__setattr__(model, fn, _Shutdown(self, fn))
        return model

    def _check_alive(self, phase: str) -> None:
        dead = [i for i, p in enumerate(self.procs) if not p.is_alive()]
        if dead:
            msgs = []
            for i in dead:
                try:
                    msgs.append(f"worker {i}: {self.out_qs[i].get_nowait()[1]}")
                except queue.Empty:
                    msgs.append(f"worker {i}: exited with code {self.procs[i].exitcode}")
            self.deparallelize()
            raise DeploymentError(f"worker(s) {dead} died during {phase}:\n" + "\n".join(msgs))

    def forward(self, fn: str, *args, **kwargs):
        if not self.procs:
            raise DeploymentError("the deployment workers have been shut down")
        args, kwargs = _strip_for_pickle(args), _strip_for_pickle(kwargs)
        for q in self.in_qs:
            q.put((fn, args, kwargs))
        results = []
        deadline = time.time() + self.request_timeout_s
        for rank, q in enumerate(self.out_qs):
            while True:
                try:
                    results.append(q.get(timeout=0.2))
                    break
                except queue.Empty:
                    self._check_alive(f"request {fn!r}")
                    if time.time() > deadline:
                        self.deparallelize()
                        raise DeploymentError(f"worker {rank} did not answer {fn!r} within {self.request_timeout_s}s")
        for rank, (kind, payload) in enumerate(results):
            if kind != "ok":
                raise DeploymentError(f"worker {rank} raised during {fn!r}:\n{payload}")
        return results[0][1]

    def deparallelize(self) -> None:
        for q in self.in_qs:
            try:
                q.put(None)
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
        self.procs, self.in_qs, self.out_qs = [], [], []


class _Proxy:
    def __init__(self, engine: DeploymentParallelEngine, fn: str) -> None:
        self.engine, self.fn = engine, fn

    def __call__(self, *args, **kwargs):
        out = self.engine.forward(self.fn, *args, **kwargs)
        return self.engine.model if self.fn == "fuse" else out     # model.fuse() switches every worker to the kernels


class _Shutdown:
    """``model.cpu()`` / ``.cuda()`` / ``.to()`` on a deployed model end the deployment (as in the reference)."""

    def __init__(self, engine: DeploymentParallelEngine, fn: str) -> None:
        self.engine, self.fn = engine, fn

    def __call__(self, *args, **kwargs):
        self.engine.deparallelize()
        model = self.engine.model
        for name in ("generate", "forward", "fuse", "cpu", "cuda", "to"):
            model.__dict__.pop(name, None)
        if self.engine.factory is not None:
            return model         # a weightless handle (the workers built the model): nothing to move
        return getattr(model, self.fn)(*args, **kwargs)
