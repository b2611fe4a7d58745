"""``GenerationMixin``: greedy, sampling, beam, beam-sampling and diverse (group) beam search.

Self-contained restatement of the generate API the reference vendors from HF
(oslo/generation_utils.py) with its four OSLO-specific behaviours kept:

* ``fused_no_repeat_ngram_blocking`` kwarg / config attribute selects the device-side n-gram blocker;
* under tensor parallelism ``input_ids`` are broadcast from the tensor-parallel source rank (the
  reference broadcasts over the world group, which is wrong once data parallelism is present);
* under pipeline parallelism the micro-batch size is set to the whole batch before each model call;
* the pipeline generator is unwrapped to its single output.

Decoding uses a static, in-place KV cache and asks the model for last-position logits only.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Union

import torch
import torch.distributed as dist
from torch import Tensor

from .beam_search import BeamSearchScorer
from .logits_process import (ForcedBOSTokenLogitsProcessor, ForcedEOSTokenLogitsProcessor,
                             FusedNoRepeatNGramLogitsProcessor, HammingDiversityLogitsProcessor,
                             InfNanRemoveLogitsProcessor, LogitsProcessorList, MaxLengthCriteria, MaxTimeCriteria,
                             MinLengthLogitsProcessor, NoBadWordsLogitsProcessor, NoRepeatNGramLogitsProcessor,
                             PrefixConstrainedLogitsProcessor, RepetitionPenaltyLogitsProcessor,
                             StoppingCriteriaList, TemperatureLogitsWarper, TopKLogitsWarper, TopPLogitsWarper)


class GenerateOutput(dict):
    """``sequences`` plus optional ``scores`` / ``sequences_scores``; attribute access like ``ModelOutput``."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e


class GenerationMixin:
    # ------------------------------------------------------------------ hooks models may override
    def prepare_inputs_for_generation(self, input_ids: Tensor, **kwargs) -> Dict[str, Any]:
        return {"input_ids": input_ids}

    def adjust_logits_during_generation(self, logits: Tensor, **kwargs) -> Tensor:
        return logits

    @staticmethod
    def _reorder_cache(past, beam_idx: Tensor):
        raise NotImplementedError("this model does not define _reorder_cache; beam search needs it")

    # ------------------------------------------------------------------ helpers
    def _gen_forward(self, model_inputs: Dict[str, Any]):
        """One model call that works with and without pipeline parallelism."""
        if getattr(self, "is_pipeline_parallelized", lambda: False)():
            ref = model_inputs.get("input_ids")
            self.set_micro_batch_size(ref.size(0))
            out = self(**model_inputs, return_dict=True, last_token_logits=True)
            return [o for o in out][0]
        return self(**model_inputs, return_dict=True, last_token_logits=True)

    @staticmethod
    def _update_model_kwargs_for_generation(outputs, model_kwargs: Dict[str, Any]) -> Dict[str, Any]:
        past = None
        if hasattr(outputs, "get"):
            past = outputs.get("past_key_values")
        if past is not None:
            model_kwargs["past_key_values"] = past
        am = model_kwargs.get("attention_mask")
        if am is not None:
            model_kwargs["attention_mask"] = torch.cat([am, am.new_ones((am.shape[0], 1))], dim=-1)
        tt = model_kwargs.get("token_type_ids")
        if tt is not None:
            model_kwargs["token_type_ids"] = torch.cat([tt, tt[:, -1:]], dim=-1)
        return model_kwargs

    @staticmethod
    def _expand_inputs_for_generation(input_ids: Tensor, expand_size: int, **model_kwargs):
        idx = torch.arange(input_ids.shape[0], device=input_ids.device).view(-1, 1).repeat(1, expand_size).view(-1)
        input_ids = input_ids.index_select(0, idx)
        for k in ("attention_mask", "token_type_ids", "position_ids"):
            if model_kwargs.get(k) is not None:
                model_kwargs[k] = model_kwargs[k].index_select(0, idx)
        return input_ids, model_kwargs

    def _get_logits_processor(self, repetition_penalty, no_repeat_ngram_size, bad_words_ids, min_length, max_length,
                              eos_token_id, forced_bos_token_id, forced_eos_token_id, prefix_allowed_tokens_fn,
                              num_beams, num_beam_groups, diversity_penalty, remove_invalid_values,
                              fused_no_repeat_ngram_blocking) -> LogitsProcessorList:
        procs = LogitsProcessorList()
        if diversity_penalty is not None and diversity_penalty > 0.0:
            procs.append(HammingDiversityLogitsProcessor(diversity_penalty, num_beams, num_beam_groups))
        if repetition_penalty is not None and repetition_penalty != 1.0:
            procs.append(RepetitionPenaltyLogitsProcessor(repetition_penalty))
        if no_repeat_ngram_size is not None and no_repeat_ngram_size > 0:
            cls = FusedNoRepeatNGramLogitsProcessor if fused_no_repeat_ngram_blocking else NoRepeatNGramLogitsProcessor
            procs.append(cls(no_repeat_ngram_size))
        if bad_words_ids is not None:
            procs.append(NoBadWordsLogitsProcessor(bad_words_ids, eos_token_id))
        if min_length is not None and eos_token_id is not None and min_length > 0:
            procs.append(MinLengthLogitsProcessor(min_length, eos_token_id))
        if prefix_allowed_tokens_fn is not None:
            procs.append(PrefixConstrainedLogitsProcessor(prefix_allowed_tokens_fn, num_beams // num_beam_groups))
        if forced_bos_token_id is not None:
            procs.append(ForcedBOSTokenLogitsProcessor(forced_bos_token_id))
        if forced_eos_token_id is not None:
            procs.append(ForcedEOSTokenLogitsProcessor(max_length, forced_eos_token_id))
        if remove_invalid_values:
            procs.append(InfNanRemoveLogitsProcessor())
        return procs

    @staticmethod
    def _get_logits_warper(top_k, top_p, temperature, num_beams) -> LogitsProcessorList:
        warpers = LogitsProcessorList()
        keep = 2 if num_beams > 1 else 1
        if temperature is not None and temperature != 1.0:
            warpers.append(TemperatureLogitsWarper(temperature))
        if top_k is not None and top_k != 0:
            warpers.append(TopKLogitsWarper(top_k, min_tokens_to_keep=keep))
        if top_p is not None and top_p < 1.0:
            warpers.append(TopPLogitsWarper(top_p, min_tokens_to_keep=keep))
        return warpers

    # ------------------------------------------------------------------ entry point
    @torch.no_grad()
    def generate(self, input_ids: Optional[Tensor] = None, max_length: Optional[int] = None,
                 min_length: Optional[int] = None, do_sample: Optional[bool] = None,
                 early_stopping: Optional[bool] = None, num_beams: Optional[int] = None,
                 temperature: Optional[float] = None, top_k: Optional[int] = None, top_p: Optional[float] = None,
                 repetition_penalty: Optional[float] = None, bad_words_ids: Optional[List[List[int]]] = None,
                 bos_token_id: Optional[int] = None, pad_token_id: Optional[int] = None,
                 eos_token_id: Optional[int] = None, length_penalty: Optional[float] = None,
                 no_repeat_ngram_size: Optional[int] = None, encoder_no_repeat_ngram_size: Optional[int] = None,
                 num_return_sequences: Optional[int] = None,
                 max_time: Optional[float] = None, max_new_tokens: Optional[int] = None,
                 decoder_start_token_id: Optional[int] = None,
                 use_cache: Optional[bool] = None, num_beam_groups: Optional[int] = None,
                 diversity_penalty: Optional[float] = None,
                 prefix_allowed_tokens_fn: Optional[Callable[[int, Tensor], List[int]]] = None,
                 output_attentions: Optional[bool] = None, output_hidden_states: Optional[bool] = None,
                 output_scores: bool = False, return_dict_in_generate: bool = False,
                 forced_bos_token_id: Optional[int] = None, forced_eos_token_id: Optional[int] = None,
                 remove_invalid_values: Optional[bool] = None, synced_gpus: bool = False,
                 fused_no_repeat_ngram_blocking: Optional[bool] = None, use_static_cache: bool = True,
                 cuda_graph: bool = False, **model_kwargs) -> Union[Tensor, GenerateOutput]:
        """``cuda_graph=True`` (not in the reference) runs plain greedy decoding - one beam, no sampling, no logits
        processors, no attention mask - through ``GraphedGreedyDecoder``: eager prefill, then one CUDA-graph replay per
        token. Any other combination ignores the flag.

        ``output_attentions`` / ``output_hidden_states`` with ``return_dict_in_generate=True`` add ``attentions`` /
        ``hidden_states`` to the result: one entry per generated token, each a tuple over the layers, as the reference's
        decoder-only outputs do (oslo/generation_utils.py:53-121). ``encoder_no_repeat_ngram_size`` and
        ``decoder_start_token_id`` exist in the signature for call compatibility; they only mean something for
        encoder-decoder models, which this package (like the reference's model zoo) does not have."""
        cfg = self.config

        def pick(v, name, default=None):
            return v if v is not None else getattr(cfg, name, default)

        num_beams = pick(num_beams, "num_beams", 1)
        num_beam_groups = pick(num_beam_groups, "num_beam_groups", 1)
        do_sample = pick(do_sample, "do_sample", False)
        num_return_sequences = pick(num_return_sequences, "num_return_sequences", 1)
        pad_token_id = pick(pad_token_id, "pad_token_id")
        bos_token_id = pick(bos_token_id, "bos_token_id")
        eos_token_id = pick(eos_token_id, "eos_token_id")
        min_length = pick(min_length, "min_length", 0)
        early_stopping = pick(early_stopping, "early_stopping", False)
        length_penalty = pick(length_penalty, "length_penalty", 1.0)
        repetition_penalty = pick(repetition_penalty, "repetition_penalty", 1.0)
        no_repeat_ngram_size = pick(no_repeat_ngram_size, "no_repeat_ngram_size", 0)
        diversity_penalty = pick(diversity_penalty, "diversity_penalty", 0.0)
        use_cache = pick(use_cache, "use_cache", True)
        fused_ngram = pick(fused_no_repeat_ngram_blocking, "fused_no_repeat_ngram_blocking", False)
        if do_sample:
            temperature = pick(temperature, "temperature", 1.0)
            top_k = pick(top_k, "top_k", 50)
            top_p = pick(top_p, "top_p", 1.0)
        if pad_token_id is None and eos_token_id is not None:
            pad_token_id = eos_token_id

        if input_ids is None:
            if bos_token_id is None:
                raise ValueError("input_ids or bos_token_id is required")
            input_ids = torch.full((1, 1), bos_token_id, dtype=torch.long, device=self.device)
        input_ids = input_ids.to(self.device)
        mpu = getattr(self, "mpu", None)
        if mpu is not None and mpu.get_tensor_parallel_world_size() > 1 and dist.is_initialized():
            input_ids = input_ids.contiguous()
            dist.broadcast(input_ids, src=mpu.get_tensor_parallel_src_rank(), group=mpu.get_tensor_parallel_group())
        if model_kwargs.get("attention_mask") is None and pad_token_id is not None and \
                bool((input_ids == pad_token_id).any()) and pad_token_id != eos_token_id:
            model_kwargs["attention_mask"] = input_ids.ne(pad_token_id).long()
        elif model_kwargs.get("attention_mask") is not None:
            model_kwargs["attention_mask"] = model_kwargs["attention_mask"].to(self.device)

        cur_len = input_ids.shape[-1]
        if max_new_tokens is not None:
            max_length = cur_len + max_new_tokens
        max_length = pick(max_length, "max_length", 20)
        if cur_len >= max_length:
            raise ValueError(f"input length {cur_len} is not shorter than max_length {max_length}")

        is_group = num_beam_groups > 1
        if is_group and do_sample:
            raise ValueError("diverse beam search cannot be combined with sampling")
        if num_beam_groups > num_beams:
            raise ValueError("num_beam_groups must be <= num_beams")
        model_kwargs["use_cache"] = use_cache
        want_att = bool(pick(output_attentions, "output_attentions", False))
        want_hid = bool(pick(output_hidden_states, "output_hidden_states", False))
        if return_dict_in_generate and (want_att or want_hid):
            model_kwargs["_gen_trace"] = {"attentions": [] if want_att else None, "hidden_states": [] if want_hid else None}
            cuda_graph = False                         # the captured step returns token ids only
        if use_cache and use_static_cache and model_kwargs.get("past_key_values") is None:
            from ..models.common import StaticKVCache
            model_kwargs["past_key_values"] = StaticKVCache(max_length)

        procs = self._get_logits_processor(
            repetition_penalty, no_repeat_ngram_size, bad_words_ids, min_length, max_length, eos_token_id,
            forced_bos_token_id, forced_eos_token_id, prefix_allowed_tokens_fn, num_beams, num_beam_groups,
            diversity_penalty, remove_invalid_values, fused_ngram)
        stops = StoppingCriteriaList([MaxLengthCriteria(max_length)])
        if max_time is not None:
            stops.append(MaxTimeCriteria(max_time))
        common = dict(pad_token_id=pad_token_id, eos_token_id=eos_token_id, output_scores=output_scores,
                      return_dict_in_generate=return_dict_in_generate, synced_gpus=synced_gpus)

        if num_beams == 1 and not do_sample:
            if num_return_sequences > 1:
                raise ValueError("greedy search returns one sequence; use sampling or beams")
            if (cuda_graph and len(procs) == 0 and model_kwargs.get("attention_mask") is None and not output_scores
                    and max_time is None and use_cache and not getattr(self, "is_pipeline_parallelized", lambda: False)()):
                return self._graph_greedy(input_ids, max_length, pad_token_id, eos_token_id, return_dict_in_generate)
            return self.greedy_search(input_ids, procs, stops, **common, **model_kwargs)
        if num_beams == 1 and do_sample:
            warper = self._get_logits_warper(top_k, top_p, temperature, num_beams)
            input_ids, model_kwargs = self._expand_inputs_for_generation(input_ids, num_return_sequences, **model_kwargs)
            return self.sample(input_ids, procs, stops, warper, **common, **model_kwargs)
        bsz = input_ids.shape[0]
        if num_return_sequences > num_beams:
            raise ValueError("num_return_sequences must be <= num_beams")
        scorer = BeamSearchScorer(bsz, num_beams, self.device, length_penalty, early_stopping,
                                  num_return_sequences, num_beam_groups, max_length)
        input_ids, model_kwargs = self._expand_inputs_for_generation(input_ids, num_beams, **model_kwargs)
        if is_group:
            return self.group_beam_search(input_ids, scorer, procs, stops, **common, **model_kwargs)
        if do_sample:
            warper = self._get_logits_warper(top_k, top_p, temperature, num_beams)
            return self.beam_sample(input_ids, scorer, procs, stops, warper, **common, **model_kwargs)
        return self.beam_search(input_ids, scorer, procs, stops, **common, **model_kwargs)

    def _graph_greedy(self, input_ids, max_length, pad_token_id, eos_token_id, return_dict):
        """Greedy search through the CUDA-graph decoder; rows that hit ``eos_token_id`` are padded afterwards and
        the result is cut where the slowest row finished, which is what ``greedy_search`` returns."""
        from .graph_decode import GraphedGreedyDecoder
        dec = getattr(self, "_graph_decoder", None)
        if dec is None or dec.max_len < max_length:
            dec = GraphedGreedyDecoder(self, max_len=max_length)
            object.__setattr__(self, "_graph_decoder", dec)
        cur_len = input_ids.shape[-1]
        seq = dec.generate(input_ids, max_length - cur_len)
        if eos_token_id is not None:
            new = seq[:, cur_len:]
            is_eos = new == eos_token_id
            after = (is_eos.long().cumsum(dim=1) - is_eos.long()) > 0      # strictly after the first eos of the row
            new = new.masked_fill(after, pad_token_id)
            done_at = torch.where(is_eos.any(dim=1), is_eos.long().argmax(dim=1) + 1,
                                  torch.full_like(is_eos[:, 0], new.size(1), dtype=torch.long))
            keep = int(done_at.max())
            seq = torch.cat([seq[:, :cur_len], new[:, :keep]], dim=1)
        return self._finish(seq, None, return_dict)

    # ------------------------------------------------------------------ search loops
    def _all_done(self, finished_here: bool, synced_gpus: bool) -> bool:
        if not synced_gpus or not dist.is_initialized():
            return finished_here
        flag = torch.tensor(0.0 if finished_here else 1.0, device=self.device)
        dist.all_reduce(flag)
        return flag.item() == 0.0

    def _step_logits(self, input_ids, model_kwargs):
        inputs = self.prepare_inputs_for_generation(input_ids, **model_kwargs)
        trace = model_kwargs.get("_gen_trace")
        if trace is not None:
            inputs["output_attentions"] = trace["attentions"] is not None
            inputs["output_hidden_states"] = trace["hidden_states"] is not None
        out = self._gen_forward(inputs)
        if trace is not None:
            for key in ("attentions", "hidden_states"):
                if trace[key] is not None:
                    trace[key].append(out.get(key) if hasattr(out, "get") else None)
        logits = out["logits"][:, -1, :].float()
        return out, logits

    @staticmethod
    def _traced(model_kwargs) -> Dict[str, Any]:
        """``attentions`` / ``hidden_states`` collected by ``_step_logits`` (one tuple over the layers per step)."""
        trace = model_kwargs.get("_gen_trace") or {}
        return {k: tuple(v) for k, v in trace.items() if v is not None}

    def _finish(self, sequences, scores, return_dict, **extra):
        if return_dict:
            return GenerateOutput(sequences=sequences, scores=tuple(scores) if scores is not None else None, **extra)
        return sequences

    def greedy_search(self, input_ids, logits_processor=None, stopping_criteria=None, pad_token_id=None,
                      eos_token_id=None, output_scores=False, return_dict_in_generate=False, synced_gpus=False,
                      **model_kwargs):
        procs = logits_processor or LogitsProcessorList()
        stops = stopping_criteria or StoppingCriteriaList()
        scores = [] if (return_dict_in_generate and output_scores) else None
        unfinished = input_ids.new_ones(input_ids.shape[0])
        while True:
            out, logits = self._step_logits(input_ids, model_kwargs)
            s = procs(input_ids, logits)
            if scores is not None:
                scores.append(s)
            nxt = torch.argmax(s, dim=-1)
            if eos_token_id is not None:
                nxt = nxt * unfinished + pad_token_id * (1 - unfinished)
                unfinished = unfinished.mul((nxt != eos_token_id).long())
            input_ids = torch.cat([input_ids, nxt[:, None]], dim=-1)
            model_kwargs = self._update_model_kwargs_for_generation(out, model_kwargs)
            done = bool(unfinished.max() == 0) or stops(input_ids, scores)
            if self._all_done(done, synced_gpus):
                break
        return self._finish(input_ids, scores, return_dict_in_generate, **self._traced(model_kwargs))

    def sample(self, input_ids, logits_processor=None, stopping_criteria=None, logits_warper=None,
               pad_token_id=None, eos_token_id=None, output_scores=False, return_dict_in_generate=False,
               synced_gpus=False, **model_kwargs):
        procs = logits_processor or LogitsProcessorList()
        stops = stopping_criteria or StoppingCriteriaList()
        warper = logits_warper or LogitsProcessorList()
        scores = [] if (return_dict_in_generate and output_scores) else None
        unfinished = input_ids.new_ones(input_ids.shape[0])
        while True:
            out, logits = self._step_logits(input_ids, model_kwargs)
            s = warper(input_ids, procs(input_ids, logits))
            if scores is not None:
                scores.append(s)
            nxt = torch.multinomial(torch.softmax(s, dim=-1), num_samples=1).squeeze(1)
            if eos_token_id is not None:
                nxt = nxt * unfinished + pad_token_id * (1 - unfinished)
                unfinished = unfinished.mul((nxt != eos_token_id).long())
            input_ids = torch.cat([input_ids, nxt[:, None]], dim=-1)
            model_kwargs = self._update_model_kwargs_for_generation(out, model_kwargs)
            done = bool(unfinished.max() == 0) or stops(input_ids, scores)
            if self._all_done(done, synced_gpus):
                break
        return self._finish(input_ids, scores, return_dict_in_generate, **self._traced(model_kwargs))

    def _beam_loop(self, input_ids, scorer: BeamSearchScorer, procs, stops, warper, sample: bool, pad_token_id,
                   eos_token_id, output_scores, return_dict_in_generate, synced_gpus, model_kwargs):
        bsz, nb = len(scorer._hyps), scorer.num_beams
        if bsz * nb != input_ids.shape[0]:
            raise ValueError("input_ids must hold batch_size * num_beams rows")
        cur_len = input_ids.shape[-1]
        beam_scores = torch.zeros((bsz, nb), dtype=torch.float, device=input_ids.device)
        if not sample:
            beam_scores[:, 1:] = -1e9
        beam_scores = beam_scores.view(-1)
        scores = [] if (return_dict_in_generate and output_scores) else None
        while True:
            out, logits = self._step_logits(input_ids, model_kwargs)
            logits = self.adjust_logits_during_generation(logits, cur_len=cur_len)
            lp = torch.log_softmax(logits, dim=-1)
            lp = procs(input_ids, lp) + beam_scores[:, None]
            if warper is not None:
                lp = warper(input_ids, lp)
            if scores is not None:
                scores.append(lp)
            vocab = lp.shape[-1]
            lp = lp.view(bsz, nb * vocab)
            if sample:
                probs = torch.softmax(lp, dim=-1)
                nt = torch.multinomial(probs, num_samples=2 * nb)
                ns = torch.gather(lp, -1, nt)
                ns, order = torch.sort(ns, descending=True, dim=1)
                nt = torch.gather(nt, -1, order)
            else:
                ns, nt = torch.topk(lp, 2 * nb, dim=1, largest=True, sorted=True)
            ni = torch.div(nt, vocab, rounding_mode="floor")
            nt = nt % vocab
            res = scorer.process(input_ids, ns, nt, ni, pad_token_id=pad_token_id, eos_token_id=eos_token_id)
            beam_scores, btok, bidx = res["next_beam_scores"], res["next_beam_tokens"], res["next_beam_indices"]
            input_ids = torch.cat([input_ids[bidx, :], btok.unsqueeze(-1)], dim=-1)
            model_kwargs = self._update_model_kwargs_for_generation(out, model_kwargs)
            if model_kwargs.get("past_key_values") is not None:
                model_kwargs["past_key_values"] = self._reorder_cache(model_kwargs["past_key_values"], bidx)
            cur_len += 1
            done = scorer.is_done or stops(input_ids, scores)
            if self._all_done(done, synced_gpus):
                break
        fin = scorer.finalize(input_ids, beam_scores, stops.max_length or cur_len, pad_token_id, eos_token_id)
        return self._finish(fin["sequences"], scores, return_dict_in_generate, sequences_scores=fin["sequence_scores"],
                            **self._traced(model_kwargs))

    def beam_search(self, input_ids, beam_scorer, logits_processor=None, stopping_criteria=None, pad_token_id=None,
                    eos_token_id=None, output_scores=False, return_dict_in_generate=False, synced_gpus=False,
                    **model_kwargs):
        return self._beam_loop(input_ids, beam_scorer, logits_processor or LogitsProcessorList(),
                               stopping_criteria or StoppingCriteriaList(), None, False, pad_token_id, eos_token_id,
                               output_scores, return_dict_in_generate, synced_gpus, model_kwargs)

    def beam_sample(self, input_ids, beam_scorer, logits_processor=None, stopping_criteria=None, logits_warper=None,
                    pad_token_id=None, eos_token_id=None, output_scores=False, return_dict_in_generate=False,
                    synced_gpus=False, **model_kwargs):
        return self._beam_loop(input_ids, beam_scorer, logits_processor or LogitsProcessorList(),
                               stopping_criteria or StoppingCriteriaList(), logits_warper or LogitsProcessorList(),
                               True, pad_token_id, eos_token_id, output_scores, return_dict_in_generate,
                               synced_gpus, model_kwargs)

    def group_beam_search(self, input_ids, beam_scorer: BeamSearchScorer, logits_processor=None,
                          stopping_criteria=None, pad_token_id=None, eos_token_id=None, output_scores=False,
                          return_dict_in_generate=False, synced_gpus=False, **model_kwargs):
        procs = logits_processor or LogitsProcessorList()
        stops = stopping_criteria or StoppingCriteriaList()
        bsz, nb = len(beam_scorer._hyps), beam_scorer.num_beams
        ng, gs = beam_scorer.num_beam_groups, beam_scorer.group_size
        dev = input_ids.device
        cur_len = input_ids.shape[-1]
        beam_scores = torch.full((bsz, nb), -1e9, dtype=torch.float, device=dev)
        beam_scores[:, ::gs] = 0
        beam_scores = beam_scores.view(-1)
        scores = [] if (return_dict_in_generate and output_scores) else None
        while True:
            current_tokens = torch.zeros(bsz * nb, dtype=input_ids.dtype, device=dev)
            reorder = torch.zeros(bsz * nb, dtype=torch.long, device=dev)
            out, logits_all = self._step_logits(input_ids, model_kwargs)
            step_scores = torch.zeros_like(logits_all) if scores is not None else None
            for g in range(ng):
                lo, hi = g * gs, min(g * gs + gs, nb)
                rows = torch.tensor([b * nb + i for b in range(bsz) for i in range(lo, hi)], device=dev)
                gin = input_ids[rows]
                lp = torch.log_softmax(logits_all[rows], dim=-1)
                vocab = lp.shape[-1]
                lp = procs(gin, lp, current_tokens=current_tokens, beam_group_idx=g)
                lp = lp + beam_scores[rows].unsqueeze(-1)
                if step_scores is not None:
                    step_scores[rows] = lp
                lp = lp.view(bsz, (hi - lo) * vocab)
                ns, nt = torch.topk(lp, 2 * (hi - lo), dim=1, largest=True, sorted=True)
                ni = torch.div(nt, vocab, rounding_mode="floor")
                nt = nt % vocab
                res = beam_scorer.process(gin, ns, nt, ni, pad_token_id=pad_token_id, eos_token_id=eos_token_id)
                beam_scores[rows] = res["next_beam_scores"]
                btok, bidx = res["next_beam_tokens"], res["next_beam_indices"]
                input_ids[rows] = gin[bidx]
                gin = torch.cat([gin[bidx, :], btok.unsqueeze(-1)], dim=-1)
                current_tokens[rows] = gin[:, -1]
                reorder[rows] = nb * torch.div(bidx, hi - lo, rounding_mode="floor") + lo + (bidx % (hi - lo))
            if scores is not None:
                scores.append(step_scores)
            input_ids = torch.cat([input_ids, current_tokens.unsqueeze(-1)], dim=-1)
            model_kwargs = self._update_model_kwargs_for_generation(out, model_kwargs)
            if model_kwargs.get("past_key_values") is not None:
                model_kwargs["past_key_values"] = self._reorder_cache(model_kwargs["past_key_values"], reorder)
            cur_len += 1
            done = beam_scorer.is_done or stops(input_ids, scores)
            if self._all_done(done, synced_gpus):
                break
        fin = beam_scorer.finalize(input_ids, beam_scores, stops.max_length or cur_len, pad_token_id, eos_token_id)
        return self._finish(fin["sequences"], scores, return_dict_in_generate, sequences_scores=fin["sequence_scores"],
                            **self._traced(model_kwargs))
