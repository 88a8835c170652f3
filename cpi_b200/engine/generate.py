"""The generation loop above the step function.

Reference loop for one prompt (src/engine/llama4_cuda_engine.cu:541-621): run the prompt, then
repeat { sample; append; stop if the token is the end token (it is kept in the output); stop if the
callback says so; stop at max_new; stop when the context is full; run the token }.  Here the same order
of decisions holds per sequence, for batches of unequal prompts that start together: a sequence that
stops leaves the next step's batch and gives its slot back at once, and when more requests are given
than fit, batch follows batch in slots that the previous one freed.

The loop talks to the engine through four calls (acquire_slot, release_slot, step, length) and to a
sampler through one, so its decisions can be tested without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..sampling.params import SamplingParams, GREEDY


@dataclass
class GenerationRequest:
    prompt: Sequence[int]
    max_new: int = 16
    sampling: SamplingParams = GREEDY
    stop_ids: Optional[Sequence[int]] = None      # None: the model's own end tokens


@dataclass
class GenerationResult:
    tokens: list                                   # generated ids (the prompt is not repeated)
    finish_reason: str                             # "stop_token" | "max_new" | "capacity" | "callback"
    prompt_tokens: int


@dataclass
class GenerationStats:
    """Wall-clock phases like the reference's BenchmarkStats (include/engine/llama_engine.hpp:102-127)."""
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    batches: int = 0
    decode_steps: int = 0


def _rounded(n: int, page: int) -> int:
    return -(-n // page) * page


def plan_batches(requests: Sequence[GenerationRequest], *, max_batch: int, token_capacity: int, page_size: int,
                 max_seq_len: int) -> list:
    """Splits request indices, in order, into batches that fit: at most max_batch sequences, and the sum
    of each sequence's most tokens (prompt + max_new - 1 cached positions, rounded up to pages) within
    the cache.  A request that cannot fit alone is an error."""
    batches, cur, used = [], [], 0
    for i, r in enumerate(requests):
        need = _rounded(min(len(r.prompt) + max(r.max_new - 1, 0), max_seq_len), page_size)
        if len(r.prompt) > max_seq_len:
            raise ValueError(f"request {i}: prompt of {len(r.prompt)} tokens exceeds the longest sequence "
                             f"({max_seq_len})")
        if need > token_capacity:
            raise ValueError(f"request {i}: needs {need} cached tokens, the cache holds {token_capacity}")
        if cur and (len(cur) >= max_batch or used + need > token_capacity):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class Generator:
    def __init__(self, engine, sampler, *, max_batch: int, default_stop_ids: Sequence[int] = (),
                 bos_token_id: Optional[int] = None, step_entry=None):
        self.engine, self.sampler = engine, sampler
        self.max_batch = max_batch
        self.default_stop_ids = tuple(default_stop_ids)
        self.bos_token_id = bos_token_id
        if step_entry is None:
            from .engine import StepEntry as step_entry
        self._entry = step_entry
        self.stats = GenerationStats()

    def generate(self, requests: Sequence[GenerationRequest],
                 on_token: Optional[Callable[[int, int], bool]] = None) -> list:
        """Runs every request; `on_token(request index, token)` returning False stops that request."""
        reqs = []
        for i, r in enumerate(requests):
            prompt = [int(t) for t in r.prompt]
            if not prompt:
                if self.bos_token_id is None:
                    raise ValueError(f"request {i}: empty prompt and the model names no begin-of-text token")
                prompt = [self.bos_token_id]          # as the reference does (:565-569)
            if r.max_new < 1:
                raise ValueError(f"request {i}: max_new must be >= 1")
            r.sampling.validate()
            reqs.append(GenerationRequest(prompt, r.max_new, r.sampling, r.stop_ids))
        cache = self.engine.cache
        batches = plan_batches(reqs, max_batch=self.max_batch, token_capacity=cache.n_pages * cache.page_size,
                               page_size=cache.page_size, max_seq_len=cache.max_seq_len)
        self.stats = GenerationStats()
        results: list = [None] * len(reqs)
        for batch in batches:
            self._run_batch(batch, reqs, results, on_token)
            self.stats.batches += 1
        return results

    def _run_batch(self, idxs, reqs, results, on_token):
        eng = self.engine
        max_len = eng.cache.max_seq_len
        live = list(idxs)
        slot = {i: eng.acquire_slot() for i in live}
        out = {i: [] for i in live}
        stops = {i: set(self.default_stop_ids if reqs[i].stop_ids is None else reqs[i].stop_ids) for i in live}
        t0 = time.perf_counter()
        try:
            logits = eng.step([self._entry(slot[i], reqs[i].prompt, [len(reqs[i].prompt) - 1]) for i in live])
            self.stats.prompt_tokens += sum(len(reqs[i].prompt) for i in live)
            step = 0
            t1 = None
            while live:
                toks = self.sampler.sample(logits, [reqs[i].sampling for i in live],
                                           [list(reqs[i].prompt) + out[i] for i in live],
                                           [(i, step) for i in live])
                if t1 is None:                      # the first sample ends the prefill phase
                    t1 = time.perf_counter()
                    self.stats.prefill_ms += (t1 - t0) * 1e3
                nxt = []
                for i, tok in zip(live, toks):
                    tok = int(tok)
                    out[i].append(tok)
                    self.stats.generated_tokens += 1
                    reason = None
                    if tok in stops[i]:
                        reason = "stop_token"
                    elif on_token is not None and not on_token(i, tok):
                        reason = "callback"
                    elif len(out[i]) >= reqs[i].max_new:
                        reason = "max_new"
                    elif len(reqs[i].prompt) + len(out[i]) > max_len:
                        reason = "capacity"
                    if reason is None:
                        nxt.append(i)
                    else:
                        results[i] = GenerationResult(out[i], reason, len(reqs[i].prompt))
                        eng.release_slot(slot.pop(i))
                live = nxt
                if not live:
                    break
                logits = eng.step([self._entry(slot[i], [out[i][-1]], [0]) for i in live])
                self.stats.decode_steps += 1
                step += 1
            if t1 is not None:
                self.stats.decode_ms += (time.perf_counter() - t1) * 1e3
        finally:
            for s in slot.values():                 # an error must not leak slots
                eng.release_slot(s)
