"""Chooses next tokens from logits on the device.

Order of operations, as in the reference's sampler (src/engine/llama4_cuda_engine.cu:64-225): clamp and
sanitise, repetition penalty over the distinct ids of prompt + generated tokens (only if > 1),
no-repeat-n-gram bans, then greedy arg-max (first maximum) or temperature -> softmax -> top-k by
probability -> top-p cut -> renormalise -> draw.  The uniform number of a draw is a counter-based
function of (seed, request, step), so runs repeat.
"""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import lib as K
from .params import SamplingParams


def banned_by_ngram(history: list, n: int) -> list:
    """Tokens that would complete an n-gram already present in history
    (src/engine/llama4_cuda_engine.cu:101-125)."""
    if n <= 1 or len(history) + 1 < n:
        return []
    prefix = history[len(history) - (n - 1):]
    banned = set()
    for i in range(0, len(history) - n + 1):
        if history[i:i + n - 1] == prefix:
            banned.add(history[i + n - 1])
    return sorted(banned)


def uniform_for(seed: int, request: int, step: int) -> float:
    """A float32 in [0, 1) that depends only on (seed, request, step)."""
    g = np.random.Generator(np.random.Philox(key=int(seed) & (2 ** 64 - 1), counter=[int(request), int(step), 0, 0]))
    return float(np.float32(g.random(dtype=np.float32)))


class Sampler:
    def __init__(self, device, vocab_size: int):
        self.device, self.vocab = torch.device(device), vocab_size
        self._work = None

    def _i32(self, xs):
        return torch.tensor(xs, dtype=torch.int32, device=self.device)

    def _f32(self, xs):
        return torch.tensor(xs, dtype=torch.float32, device=self.device)

    def sample(self, logits: torch.Tensor, params: list, histories: list, counters: list) -> list:
        """The chosen token ids as a list (waits for the device)."""
        return self.sample_device(logits, params, histories, counters).tolist()

    def sample_device(self, logits: torch.Tensor, params: list, histories: list, counters: list) -> torch.Tensor:
        """logits [R, V] float32 on the device (modified in place when penalties apply);
        histories[r] = prompt + generated ids of row r (None where no option of the row reads it);
        counters[r] = (request index, step).  Returns int32 [R] on the device without waiting for it."""
        R = logits.shape[0]
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if R == 0:
            return out
        if all(p.is_plain_greedy for p in params):
            K.argmax(logits, out)
            return out
        for p in params:
            p.validate()
        if any(p.repetition_penalty > 1.0 for p in params):
            ids, offs = [], [0]
            for p, h in zip(params, histories):
                if p.repetition_penalty > 1.0:
                    ids += sorted(set(h))
                offs.append(len(ids))
            if ids:
                K.repetition_penalty(logits, self._i32(ids), self._i32(offs),
                                     self._f32([p.repetition_penalty for p in params]))
        if any(p.no_repeat_ngram_size > 1 for p in params):
            ids, offs = [], [0]
            for p, h in zip(params, histories):
                ids += banned_by_ngram(h, p.no_repeat_ngram_size)
                offs.append(len(ids))
            if ids:
                K.ban_tokens(logits, self._i32(ids), self._i32(offs))
        if self._work is None or self._work.numel() < R * self.vocab:
            self._work = torch.empty(R * self.vocab, dtype=torch.float32, device=self.device)
        u = [uniform_for(p.seed, req, step) for p, (req, step) in zip(params, counters)]
        K.sample(logits, self._work, self._f32([p.temperature for p in params]),
                 self._i32([max(1, min(p.top_k, self.vocab)) for p in params]),
                 self._f32([p.top_p for p in params]), self._f32(u), out)
        return out
