"""The generation loop above the step function.

Reference loop for one prompt (src/engine/llama4_cuda_engine.cu:541-621): run the prompt, then
repeat { sample; append; hand the token to the callback (the end token too) and stop if it says so; stop
if the token is the end token (it is kept in the output); stop at max_new; stop when the context is full
(a prompt longer than max_context is an error, :549-551; pos + 1 >= max_context ends it, :602-604); run the
token }.  Here the same order
of decisions holds per sequence, for batches of unequal prompts that start together: a sequence that
stops leaves the next step's batch and gives its slot back at once, and when more requests are given
than fit, batch follows batch in slots that the previous one freed.

The loop talks to the engine through four calls (acquire_slot, release_slot, step, length) and to a
sampler through one, so its decisions can be tested without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
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
                 bos_token_id: Optional[int] = None, step_entry=None, max_context: Optional[int] = None):
        """`max_context`: the most positions a sequence may reach (the caller's own figure: the cache may
        hold a few more, since it is sized in whole pages); default: what the cache holds per sequence."""
        self.engine, self.sampler = engine, sampler
        self.max_batch = max_batch
        self.max_context = min(int(max_context), engine.cache.max_seq_len) if max_context is not None \
            else engine.cache.max_seq_len
        self.default_stop_ids = tuple(default_stop_ids)
        self.bos_token_id = bos_token_id
        if step_entry is None:
            from .engine import StepEntry as step_entry
        self._entry = step_entry
        self.stats = GenerationStats()
        # Decode steps are launched one ahead of the host: step n+1 takes its tokens from the device tensor
        # that the sampler of step n wrote, while the host is still reading step n's tokens for the stop
        # checks.  Needs nothing from the host between steps, so it is off for requests with a callback, a
        # repetition penalty or n-gram bans.
        self.pipelined = True
        self._pinned = None

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
                               page_size=cache.page_size, max_seq_len=self.max_context)
        self.stats = GenerationStats()
        results: list = [None] * len(reqs)
        check = getattr(self.engine, "check_device_errors", None)
        for batch in batches:
            self._run_batch(batch, reqs, results, on_token)
            self.stats.batches += 1
            if check is not None:       # the batch's tokens are on the host: what kernels flagged meanwhile is too
                check()
        return results

    def _run_batch(self, idxs, reqs, results, on_token):
        needs_host = on_token is not None or any(
            reqs[i].sampling.repetition_penalty > 1.0 or reqs[i].sampling.no_repeat_ngram_size > 1 for i in idxs)
        if self.pipelined and not needs_host and hasattr(self.engine, "step_decode") \
                and hasattr(self.sampler, "sample_device"):
            return self._run_batch_pipelined(idxs, reqs, results)
        eng = self.engine
        max_len = self.max_context
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
                params = [reqs[i].sampling for i in live]
                # the histories (prompt + generated ids) are only looked at by the penalties and the n-gram bans
                need_hist = any(p.repetition_penalty > 1.0 or p.no_repeat_ngram_size > 1 for p in params)
                hist = [list(reqs[i].prompt) + out[i] for i in live] if need_hist else [None] * len(live)
                toks = self.sampler.sample(logits, params, hist, [(i, step) for i in live])
                if t1 is None:                      # the first sample ends the prefill phase
                    t1 = time.perf_counter()
                    self.stats.prefill_ms += (t1 - t0) * 1e3
                nxt = []
                for i, tok in zip(live, toks):
                    tok = int(tok)
                    out[i].append(tok)
                    self.stats.generated_tokens += 1
                    reason = None
                    # the callback sees every token, the end token too, before the end-token check (:593-598)
                    go_on = on_token(i, tok) if on_token is not None else True
                    if tok in stops[i]:
                        reason = "stop_token"
                    elif not go_on:
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

    # ---- one step ahead --------------------------------------------------------------------------
    def _host_copy(self, toks_dev, k):
        """Starts the copy of a device token tensor to the host; returns a function that waits and lists it."""
        if not toks_dev.is_cuda:
            return toks_dev.tolist
        import torch
        if self._pinned is None or self._pinned[0].numel() < toks_dev.numel():
            n = max(self.max_batch, toks_dev.numel())
            self._pinned = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        buf = self._pinned[k % 4][:toks_dev.numel()]
        buf.copy_(toks_dev, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()

        def wait():
            ev.synchronize()
            return buf.tolist()
        return wait

    def _run_batch_pipelined(self, idxs, reqs, results):
        """The same decisions as the loop above, with the next step launched before the tokens of the last
        one are known on the host.  A request that turns out to have ended on a stop token has then been
        run for one token too many; that token is dropped and the others' results do not depend on it."""
        eng, sampler = self.engine, self.sampler
        max_len = self.max_context
        live = list(idxs)
        slot = {i: eng.acquire_slot() for i in live}
        out = {i: [] for i in live}
        stops = {i: set(self.default_stop_ids if reqs[i].stop_ids is None else reqs[i].stop_ids) for i in live}
        plen = {i: len(reqs[i].prompt) for i in live}
        t0 = time.perf_counter()
        t1 = None
        try:
            logits = eng.step([self._entry(slot[i], reqs[i].prompt, [plen[i] - 1]) for i in live])
            self.stats.prompt_tokens += sum(plen[i] for i in live)
            step = 0
            toks_dev = sampler.sample_device(logits, [reqs[i].sampling for i in live], [None] * len(live),
                                             [(i, step) for i in live])
            pending, wait = live, self._host_copy(toks_dev, step)
            while pending:
                # requests that go on after the pending token unless it is a stop token
                cont = [i for i in pending
                        if len(out[i]) + 1 < reqs[i].max_new and plen[i] + len(out[i]) + 1 <= max_len]
                nxt_dev = nxt_wait = None
                if cont:
                    sel = toks_dev
                    if len(cont) != len(pending):
                        where = {i: k for k, i in enumerate(pending)}
                        sel = toks_dev[[where[i] for i in cont]]
                    logits = eng.step_decode([slot[i] for i in cont], sel)
                    self.stats.decode_steps += 1
                    nxt_dev = sampler.sample_device(logits, [reqs[i].sampling for i in cont], [None] * len(cont),
                                                    [(i, step + 1) for i in cont])
                    nxt_wait = self._host_copy(nxt_dev, step + 1)
                toks = wait()
                if t1 is None:                      # the first tokens on the host end the prefill phase
                    t1 = time.perf_counter()
                    self.stats.prefill_ms += (t1 - t0) * 1e3
                ended = set()
                for i, tok in zip(pending, toks):
                    tok = int(tok)
                    out[i].append(tok)
                    self.stats.generated_tokens += 1
                    reason = None
                    if tok in stops[i]:
                        reason = "stop_token"
                    elif len(out[i]) >= reqs[i].max_new:
                        reason = "max_new"
                    elif plen[i] + len(out[i]) > max_len:
                        reason = "capacity"
                    if reason is not None:
                        results[i] = GenerationResult(out[i], reason, plen[i])
                        eng.release_slot(slot.pop(i))
                        ended.add(i)
                if not cont:
                    break
                keep = [k for k, i in enumerate(cont) if i not in ended]
                if len(keep) != len(cont):          # ended on a stop token: their extra token is dropped
                    full = nxt_wait
                    nxt_dev = nxt_dev[keep] if keep else None
                    nxt_wait = (lambda f=full, kk=keep: [f()[k] for k in kk])
                pending, toks_dev, wait = [cont[k] for k in keep], nxt_dev, nxt_wait
                step += 1
            if t1 is not None:
                self.stats.decode_ms += (time.perf_counter() - t1) * 1e3
        finally:
            for sl in slot.values():                # an error must not leak slots
                eng.release_slot(sl)

