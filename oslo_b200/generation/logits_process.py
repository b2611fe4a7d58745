"""Logits processors / warpers and stopping criteria used by ``generate``.

Same behaviour as the HF classes the reference vendors (oslo/generation_utils.py:338-466); the
n-gram blocker has a kernel-backed variant (reference: ``FusedNoRepeatNGramLogitsProcessor``,
oslo/fused_kernels_utils.py:492-521) that runs on the current CUDA stream for any step length.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional

import torch
from torch import Tensor

from .. import ops


class LogitsProcessor:
    def __call__(self, input_ids: Tensor, scores: Tensor) -> Tensor:
        raise NotImplementedError


class LogitsWarper(LogitsProcessor):
    pass


class LogitsProcessorList(list):
    def __call__(self, input_ids: Tensor, scores: Tensor, **kwargs) -> Tensor:
        for p in self:
            scores = p(input_ids, scores, **kwargs) if kwargs and _takes_kwargs(p) else p(input_ids, scores)
        return scores


def _takes_kwargs(p) -> bool:
    return isinstance(p, HammingDiversityLogitsProcessor)


class MinLengthLogitsProcessor(LogitsProcessor):
    def __init__(self, min_length: int, eos_token_id: int) -> None:
        if min_length < 0 or eos_token_id is None or eos_token_id < 0:
            raise ValueError("min_length and eos_token_id must be non-negative")
        self.min_length, self.eos_token_id = min_length, eos_token_id

    def __call__(self, input_ids, scores):
        if input_ids.shape[-1] < self.min_length:
            scores[:, self.eos_token_id] = -float("inf")
        return scores


class TemperatureLogitsWarper(LogitsWarper):
    def __init__(self, temperature: float) -> None:
        if not temperature > 0:
            raise ValueError("temperature must be strictly positive")
        self.temperature = temperature

    def __call__(self, input_ids, scores):
        return scores / self.temperature


class RepetitionPenaltyLogitsProcessor(LogitsProcessor):
    def __init__(self, penalty: float) -> None:
        if not penalty > 0:
            raise ValueError("penalty must be strictly positive")
        self.penalty = penalty

    def __call__(self, input_ids, scores):
        s = torch.gather(scores, 1, input_ids)
        s = torch.where(s < 0, s * self.penalty, s / self.penalty)
        scores.scatter_(1, input_ids, s)
        return scores


class TopKLogitsWarper(LogitsWarper):
    def __init__(self, top_k: int, filter_value: float = -float("inf"), min_tokens_to_keep: int = 1) -> None:
        self.top_k, self.filter_value, self.min_keep = int(top_k), filter_value, min_tokens_to_keep

    def __call__(self, input_ids, scores):
        k = min(max(self.top_k, self.min_keep), scores.size(-1))
        kth = torch.topk(scores, k)[0][..., -1, None]
        return scores.masked_fill(scores < kth, self.filter_value)


class TopPLogitsWarper(LogitsWarper):
    def __init__(self, top_p: float, filter_value: float = -float("inf"), min_tokens_to_keep: int = 1) -> None:
        if not 0 <= top_p <= 1.0:
            raise ValueError("top_p must be in [0, 1]")
        self.top_p, self.filter_value, self.min_keep = float(top_p), filter_value, min_tokens_to_keep

    def __call__(self, input_ids, scores):
        sorted_logits, sorted_idx = torch.sort(scores, descending=True)
        cum = sorted_logits.softmax(dim=-1).cumsum(dim=-1)
        remove = cum > self.top_p
        if self.min_keep > 1:
            remove[..., : self.min_keep - 1] = False
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        mask = remove.scatter(1, sorted_idx, remove)
        return scores.masked_fill(mask, self.filter_value)


class NoRepeatNGramLogitsProcessor(LogitsProcessor):
    """Host-side n-gram blocking."""

    def __init__(self, ngram_size: int) -> None:
        if ngram_size <= 0:
            raise ValueError("ngram_size must be positive")
        self.ngram_size = ngram_size

    def __call__(self, input_ids, scores):
        banned = ops.reference.banned_ngram_tokens(input_ids, self.ngram_size)
        for i, toks in enumerate(banned):
            if toks:
                scores[i, toks] = -float("inf")
        return scores


class FusedNoRepeatNGramLogitsProcessor(LogitsProcessor):
    """n-gram blocking on the device (CUDA kernel for CUDA scores, PyTorch statement on CPU)."""

    def __init__(self, ngram_size: int) -> None:
        if ngram_size <= 0:
            raise ValueError("ngram_size must be positive")
        self.ngram_size = ngram_size

    def __call__(self, input_ids, scores):
        if input_ids.size(1) + 1 < self.ngram_size:
            return scores
        if scores.dtype != torch.float32:
            out = ops.ban_repeated_ngrams(input_ids, scores.float(), self.ngram_size)
            return out.to(scores.dtype)
        return ops.ban_repeated_ngrams(input_ids, scores, self.ngram_size)


class NoBadWordsLogitsProcessor(LogitsProcessor):
    def __init__(self, bad_words_ids: List[List[int]], eos_token_id: Optional[int]) -> None:
        if not bad_words_ids or any(not isinstance(b, list) or not b for b in bad_words_ids):
            raise ValueError("bad_words_ids must be a non-empty list of non-empty lists")
        self.bad = [b for b in bad_words_ids if b != [eos_token_id]]

    def __call__(self, input_ids, scores):
        rows = input_ids.tolist()
        for i, row in enumerate(rows):
            for seq in self.bad:
                pre = seq[:-1]
                if len(pre) == 0 or (len(pre) <= len(row) and row[len(row) - len(pre):] == pre):
                    scores[i, seq[-1]] = -float("inf")
        return scores


class PrefixConstrainedLogitsProcessor(LogitsProcessor):
    def __init__(self, fn: Callable[[int, Tensor], List[int]], num_beams: int) -> None:
        self.fn, self.num_beams = fn, num_beams

    def __call__(self, input_ids, scores):
        mask = torch.full_like(scores, -float("inf"))
        for b, beams in enumerate(input_ids.view(-1, self.num_beams, input_ids.shape[-1])):
            for j, sent in enumerate(beams):
                mask[b * self.num_beams + j, self.fn(b, sent)] = 0
        return scores + mask


class ForcedBOSTokenLogitsProcessor(LogitsProcessor):
    def __init__(self, bos_token_id: int) -> None:
        self.bos_token_id = bos_token_id

    def __call__(self, input_ids, scores):
        if input_ids.shape[-1] == 1:
            keep = scores[:, self.bos_token_id].clone()
            scores[:] = -float("inf")
            scores[:, self.bos_token_id] = 0 * keep
        return scores


class ForcedEOSTokenLogitsProcessor(LogitsProcessor):
    def __init__(self, max_length: int, eos_token_id: int) -> None:
        self.max_length, self.eos_token_id = max_length, eos_token_id

    def __call__(self, input_ids, scores):
        if input_ids.shape[-1] == self.max_length - 1:
            scores[:] = -float("inf")
            scores[:, self.eos_token_id] = 0
        return scores


class InfNanRemoveLogitsProcessor(LogitsProcessor):
    def __call__(self, input_ids, scores):
        scores = torch.nan_to_num(scores, nan=0.0)
        return scores.masked_fill(scores == float("inf"), torch.finfo(scores.dtype).max)


class HammingDiversityLogitsProcessor(LogitsProcessor):
    """Group beam search: penalise tokens already chosen by earlier groups at this step."""

    def __init__(self, diversity_penalty: float, num_beams: int, num_beam_groups: int) -> None:
        if not diversity_penalty > 0.0:
            raise ValueError("diversity_penalty must be > 0")
        if num_beam_groups < 2 or num_beam_groups > num_beams:
            raise ValueError("need 2 <= num_beam_groups <= num_beams")
        self.penalty, self.num_beams = diversity_penalty, num_beams
        self.sub_beams = num_beams // num_beam_groups

    def __call__(self, input_ids, scores, current_tokens: Tensor = None, beam_group_idx: int = 0):
        bsz = current_tokens.shape[0] // self.num_beams
        start = beam_group_idx * self.sub_beams
        end = min(start + self.sub_beams, self.num_beams)
        gsize = end - start
        vocab = scores.shape[-1]
        if start == 0:
            return scores
        for b in range(bsz):
            prev = current_tokens[b * self.num_beams: b * self.num_beams + start]
            freq = torch.bincount(prev, minlength=vocab).to(scores.device)
            scores[b * gsize:(b + 1) * gsize] -= self.penalty * freq
        return scores


# ---------------------------------------------------------------------- stopping criteria
class StoppingCriteria:
    def __call__(self, input_ids: Tensor, scores: Optional[Tensor], **kwargs) -> bool:
        raise NotImplementedError


class MaxLengthCriteria(StoppingCriteria):
    def __init__(self, max_length: int) -> None:
        self.max_length = max_length

    def __call__(self, input_ids, scores, **kwargs) -> bool:
        return input_ids.shape[-1] >= self.max_length


class MaxTimeCriteria(StoppingCriteria):
    def __init__(self, max_time: float, initial_timestamp: Optional[float] = None) -> None:
        self.max_time = max_time
        self.t0 = time.time() if initial_timestamp is None else initial_timestamp

    def __call__(self, input_ids, scores, **kwargs) -> bool:
        return time.time() - self.t0 > self.max_time


class StoppingCriteriaList(list):
    def __call__(self, input_ids, scores, **kwargs) -> bool:
        return any(c(input_ids, scores) for c in self)

    @property
    def max_length(self) -> Optional[int]:
        for c in self:
            if isinstance(c, MaxLengthCriteria):
                return c.max_length
        return None


def top_k_top_p_filtering(logits: Tensor, top_k: int = 0, top_p: float = 1.0,
                          filter_value: float = -float("inf"), min_tokens_to_keep: int = 1) -> Tensor:
    if top_k > 0:
        logits = TopKLogitsWarper(top_k, filter_value, min_tokens_to_keep)(None, logits)
    if 0 <= top_p < 1.0:
        logits = TopPLogitsWarper(top_p, filter_value, min_tokens_to_keep)(None, logits)
    return logits
