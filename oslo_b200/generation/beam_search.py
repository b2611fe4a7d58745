"""Beam bookkeeping: per-sentence n-best heaps with length penalty and early stopping."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import Tensor


class BeamHypotheses:
    def __init__(self, num_beams: int, length_penalty: float, early_stopping: bool) -> None:
        self.num_beams, self.length_penalty, self.early_stopping = num_beams, length_penalty, early_stopping
        self.beams: List[Tuple[float, Tensor]] = []
        self.worst_score = 1e9

    def __len__(self) -> int:
        return len(self.beams)

    def add(self, hyp: Tensor, sum_logprobs: float) -> None:
        score = sum_logprobs / (hyp.shape[-1] ** self.length_penalty)
        if len(self) < self.num_beams or score > self.worst_score:
            self.beams.append((score, hyp))
            if len(self) > self.num_beams:
                ranked = sorted((s, i) for i, (s, _) in enumerate(self.beams))
                del self.beams[ranked[0][1]]
                self.worst_score = ranked[1][0]
            else:
                self.worst_score = min(score, self.worst_score)

    def is_done(self, best_sum_logprobs: float, cur_len: int) -> bool:
        if len(self) < self.num_beams:
            return False
        if self.early_stopping:
            return True
        return self.worst_score >= best_sum_logprobs / cur_len ** self.length_penalty


class BeamSearchScorer:
    def __init__(self, batch_size: int, num_beams: int, device, length_penalty: float = 1.0,
                 do_early_stopping: bool = False, num_beam_hyps_to_keep: int = 1, num_beam_groups: int = 1,
                 max_length: Optional[int] = None) -> None:
        if num_beams <= 1:
            raise ValueError("beam search needs num_beams > 1")
        if num_beam_groups > num_beams or num_beams % num_beam_groups:
            raise ValueError("num_beams must be a multiple of num_beam_groups")
        self.num_beams, self.device = num_beams, device
        self.length_penalty, self.do_early_stopping = length_penalty, do_early_stopping
        self.num_beam_hyps_to_keep = num_beam_hyps_to_keep
        self.num_beam_groups = num_beam_groups
        self.group_size = num_beams // num_beam_groups
        self.max_length = max_length
        self._hyps = [BeamHypotheses(num_beams, length_penalty, do_early_stopping) for _ in range(batch_size)]
        self._done = torch.tensor([False] * batch_size, dtype=torch.bool)

    @property
    def is_done(self) -> bool:
        return bool(self._done.all())

    def process(self, input_ids: Tensor, next_scores: Tensor, next_tokens: Tensor, next_indices: Tensor,
                pad_token_id: Optional[int] = None, eos_token_id: Optional[int] = None):
        cur_len = input_ids.shape[-1]
        bsz = len(self._hyps)
        gs = self.group_size
        out_scores = torch.zeros((bsz, gs), dtype=next_scores.dtype)
        out_tokens = torch.zeros((bsz, gs), dtype=torch.long)
        out_indices = torch.zeros((bsz, gs), dtype=torch.long)
        ns, nt, ni = next_scores.tolist(), next_tokens.tolist(), next_indices.tolist()
        for b, hyp in enumerate(self._hyps):
            if self._done[b]:
                if pad_token_id is None:
                    raise ValueError("pad_token_id is needed once a sentence has finished")
                out_tokens[b, :] = pad_token_id
                continue
            k = 0
            for rank, (tok, score, idx) in enumerate(zip(nt[b], ns[b], ni[b])):
                batch_beam = b * gs + idx
                if eos_token_id is not None and tok == eos_token_id:
                    if rank >= gs:
                        continue
                    hyp.add(input_ids[batch_beam].clone(), score)
                else:
                    out_scores[b, k], out_tokens[b, k], out_indices[b, k] = score, tok, batch_beam
                    k += 1
                if k == gs:
                    break
            if k < gs:
                raise ValueError("not enough non-EOS candidates to fill the beam")
            self._done[b] = self._done[b] or hyp.is_done(max(ns[b]), cur_len)
        dev = input_ids.device
        return dict(next_beam_scores=out_scores.view(-1).to(dev), next_beam_tokens=out_tokens.view(-1).to(dev),
                    next_beam_indices=out_indices.view(-1).to(dev))

    def finalize(self, input_ids: Tensor, final_beam_scores: Tensor, max_length: int,
                 pad_token_id: Optional[int] = None, eos_token_id: Optional[int] = None):
        bsz = len(self._hyps)
        fs = final_beam_scores.tolist()
        for b, hyp in enumerate(self._hyps):
            if self._done[b]:
                continue
            for j in range(self.num_beams):
                hyp.add(input_ids[b * self.num_beams + j], fs[b * self.num_beams + j])
        keep = self.num_beam_hyps_to_keep
        best: List[Tensor] = []
        best_scores = torch.zeros(bsz * keep, dtype=torch.float32)
        for b, hyp in enumerate(self._hyps):
            ranked = sorted(hyp.beams, key=lambda x: x[0])
            for j in range(keep):
                score, seq = ranked.pop()
                best.append(seq)
                best_scores[b * keep + j] = score
        sent_max = min(max(len(s) for s in best) + 1, max_length)
        decoded = input_ids.new_full((bsz * keep, sent_max), pad_token_id if pad_token_id is not None else 0)
        if min(len(s) for s in best) != max(len(s) for s in best) and pad_token_id is None:
            raise ValueError("pad_token_id is needed to pad sequences of different length")
        for i, s in enumerate(best):
            decoded[i, : len(s)] = s
            if len(s) < max_length and eos_token_id is not None and len(s) < sent_max:
                decoded[i, len(s)] = eos_token_id
        return dict(sequences=decoded, sequence_scores=best_scores.to(input_ids.device))
