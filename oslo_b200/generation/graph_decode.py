"""Greedy decoding with the single-token step replayed from a CUDA graph.

The reference decodes with a Python loop that re-launches every kernel of every layer for every token and
grows the cache with ``torch.cat`` (oslo/generation_utils.py:1269-1361, oslo/models/gptj/modeling_gptj.py:239-248).
Here the prompt is prefilled eagerly into a ``StaticKVCache``; the step "embed -> blocks -> head -> argmax ->
write token -> advance positions" keeps every position on the device, is captured once, and is replayed per
token, so a token costs one graph launch. Tensor-parallel ranks capture the same step (their NCCL collectives
are part of the graph) and replay in lock-step.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor



class GraphedGreedyDecoder:
    """``decoder = GraphedGreedyDecoder(model, max_len); ids = decoder.generate(prompt_ids, max_new_tokens)``.

    ``use_graph=None`` captures on CUDA and runs the same step eagerly elsewhere (the CPU path exists so the
    device-position bookkeeping can be tested without a GPU). Batch size and ``max_len`` are fixed by the first
    call; the cache storage and the graph are reused by later calls with the same batch size.
    """

    def __init__(self, model, max_len: int, use_graph: Optional[bool] = None, warmup_steps: int = 2) -> None:
        if getattr(model, "is_pipeline_parallelized", lambda: False)():
            raise NotImplementedError("GraphedGreedyDecoder runs one model call per token on this rank; a pipeline-"
                                      "parallel model needs the stage exchange of model.generate() instead")
        self.model = model
        self.max_len = int(max_len)
        self.use_graph = use_graph
        self.warmup_steps = max(1, int(warmup_steps))
        self.cache = None            # StaticKVCache, created on the first call
        self.graph = None
        self._batch = None
        self.replays = 0
        self.launch_counter = None   # optional callable returning the number of kernels this package has launched
        self.kernels_per_step = 0    # kernels of this package inside one captured step (needs launch_counter)
        self.record_events = False   # when set, `events` holds (start, after prefill, end) CUDA events of the last call
        self.events = None

    def release(self) -> None:
        """Drop the captured graph and the cache. Call this before the process group is destroyed: a communicator
        that is still referenced by a captured graph does not shut down."""
        self.graph = None
        self.cache = None
        self._batch = None

    # ------------------------------------------------------------------ one decode step, positions on the device
    def _step(self) -> None:
        cache = self.cache
        pos = cache.lengths_dev.to(torch.long).unsqueeze(1)
        out = self.model(input_ids=self.cur, past_key_values=cache, position_ids=pos, use_cache=True,
                         return_dict=True, last_token_logits=True)
        nxt = out["logits"][:, -1, :].float().argmax(dim=-1)
        self.tokens.index_copy_(1, self.step_idx, nxt[:, None])
        self.step_idx.add_(1)
        self.cur.copy_(nxt[:, None])

    @torch.no_grad()
    def generate(self, input_ids: Tensor, max_new_tokens: int) -> Tensor:
        model = self.model
        was_training = model.training
        model.eval()
        try:
            return self._generate(input_ids, int(max_new_tokens))
        finally:
            model.train(was_training)

    def _generate(self, input_ids: Tensor, n_new: int) -> Tensor:
        b, prompt = input_ids.shape
        if prompt + n_new > self.max_len:
            raise ValueError(f"prompt {prompt} + {n_new} new tokens exceeds max_len {self.max_len}")
        dev = input_ids.device
        graph_ok = dev.type == "cuda" if self.use_graph is None else bool(self.use_graph)
        if self.cache is None or self._batch != b:
            from ..models.common import StaticKVCache  # late import: models import this package
            self.cache = StaticKVCache(self.max_len)
            self.graph = None
            self._batch = b
            self.cur = torch.zeros(b, 1, dtype=torch.long, device=dev)
            self.tokens = torch.zeros(b, self.max_len, dtype=torch.long, device=dev)
            self.step_idx = torch.zeros(1, dtype=torch.long, device=dev)
        cache = self.cache
        cache.reset()
        ev = None
        if self.record_events and dev.type == "cuda":
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
        # ---- prefill (eager; the flash kernel, host-side positions)
        out = self.model(input_ids=input_ids, past_key_values=cache, use_cache=True, return_dict=True,
                         last_token_logits=True)
        first = out["logits"][:, -1, :].float().argmax(dim=-1)
        cache.use_device_positions(True)
        self.cur.copy_(first[:, None])
        self.tokens.zero_()
        self.tokens[:, 0] = first
        self.step_idx.fill_(1)
        done = 1
        if ev is not None:
            ev[1].record()
        if graph_ok and self.graph is None and n_new - done > self.warmup_steps:
            # real steps as warm-up on a side stream, then capture (capturing does not execute the step)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(self.warmup_steps):
                    self._step()
                    done += 1
            torch.cuda.current_stream(dev).wait_stream(side)
            host_len = cache.length
            self.graph = torch.cuda.CUDAGraph()
            c0 = self.launch_counter() if self.launch_counter else 0
            with torch.cuda.graph(self.graph):
                self._step()
            self.kernels_per_step = (self.launch_counter() - c0) if self.launch_counter else 0
            cache.length = host_len  # the host-side counter moved during capture although nothing ran
        while done < n_new:
            if graph_ok and self.graph is not None:
                self.graph.replay()
                cache.length += 1
                self.replays += 1
            else:
                self._step()
            done += 1
        cache.use_device_positions(False)
        if ev is not None:
            ev[2].record()
            self.events = ev
        return torch.cat([input_ids, self.tokens[:, :n_new]], dim=1)
