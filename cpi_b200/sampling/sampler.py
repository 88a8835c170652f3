"""Chooses next tokens from logits on the device.

Order of operations, as in the reference's sampler (src/engine/llama4_cuda_engine.cu:64-225): clamp and
sanitise, repetition penalty over the distinct ids of prompt + generated tokens (only if > 1),
no-repeat-n-gram bans, then greedy arg-max (first maximum) or temperature -> softmax -> top-k by
probability -> top-p cut -> renormalise -> draw.  The uniform number of a draw is a counter-based
function of (seed, request, step), so runs repeat.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K


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


_M64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    """The finaliser of SplitMix64: a bijection of 64-bit integers that spreads every input bit."""
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, request: int, step: int) -> float:
    """A float32 in [0, 1) that depends only on (seed, request, step): a counter-based draw (three chained
    64-bit mixes, the top 24 bits), so that a run repeats from its seed whatever else was in the batch.
    Plain integer arithmetic: it is computed for every row of every step on the host."""
    x = _mix64(int(seed) & _M64)
    x = _mix64(x ^ (int(request) & _M64))
    x = _mix64(x ^ (int(step) & _M64))
    return (x >> 40) * (1.0 / (1 << 24))


class Sampler:
    def __init__(self, device, vocab_size: int):
        self.device, self.vocab = torch.device(device), vocab_size
        self._work = None
        self._stage = None         # pinned host rows (temperature, top-k, top-p, uniform) and their device twin
        self._stage_k = 0

    def _staged(self, temperature, top_k, top_p, uniform):
        """The four per-row parameter arrays on the device through one copy from pinned memory."""
        R = len(temperature)
        if self.device.type != "cuda":
            return (self._f32(temperature), self._i32(top_k), self._f32(top_p), self._f32(uniform))
        if self._stage is None or self._stage[0][0].shape[1] < R:
            n = max(64, R)
            ring = [torch.empty((4, n), dtype=torch.float32, pin_memory=True) for _ in range(4)]
            self._stage = (ring, torch.empty((4, 4, n), dtype=torch.float32, device=self.device),
                           [torch.cuda.Event() for _ in range(4)])
            self._stage_k = 0
        ring, dev, events = self._stage
        j = self._stage_k % 4
        self._stage_k += 1
        if self._stage_k > 4:
            events[j].synchronize()                      # the copy that last read this pinned buffer is done
        host = ring[j]
        host[0, :R] = torch.tensor(temperature, dtype=torch.float32)
        host[1, :R] = torch.tensor(top_k, dtype=torch.int32).view(torch.float32)
        host[2, :R] = torch.tensor(top_p, dtype=torch.float32)
        host[3, :R] = torch.tensor(uniform, dtype=torch.float32)
        d = dev[j]
        d.copy_(host, non_blocking=True)
        events[j].record()
        return d[0, :R], d[1, :R].view(torch.int32), d[2, :R], d[3, :R]

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
        t, k, tp, ud = self._staged([p.temperature for p in params],
                                    [max(1, min(p.top_k, self.vocab)) for p in params],
                                    [p.top_p for p in params], u)
        K.sample(logits, self._work, t, k, tp, ud, out)
        return out
