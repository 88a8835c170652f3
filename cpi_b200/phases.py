"""Per-phase device timings of a step, off by default.

The reference's `--benchmark-phases` reports where a decode step's time goes: rmsnorm, qkv, kv_store,
attention, wo, mlp, moe_router, moe_expert, moe_merge, lm_head (src/app/main_modes.cpp:576-617; the
counters are `BenchmarkStats::decode_*_ms`, include/engine/llama_engine.hpp:102-127).  Here a part
brackets its launches with `with phase("qkv"):`; while no timer is installed that is a shared no-op
object.  With a timer installed every bracket records two CUDA events on the current stream, and the
engine runs steps eagerly and on one stream (a replayed graph or a side stream has no place to put
the events), so the sum of the phases is more than the time of an unprofiled step: the figures say
where the time goes, not how long a step takes.
"""
from __future__ import annotations

import torch


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _Null()
_timer = None


class _Span:
    __slots__ = ("timer", "name", "start")

    def __init__(self, timer, name):
        self.timer, self.name = timer, name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self.timer.pending.append((self.timer.kind, self.name, self.start, end))
        return False


class PhaseTimer:
    """Collects (kind of step, phase) -> milliseconds; `kind` is set by the engine before each step."""

    def __init__(self):
        self.kind = "decode"
        self.pending = []
        self.ms = {}

    def collect(self) -> dict:
        """Waits for the device and folds the finished brackets into the totals; returns {kind: {phase: ms}}."""
        if self.pending:
            torch.cuda.synchronize()
            for kind, name, a, b in self.pending:
                d = self.ms.setdefault(kind, {})
                d[name] = d.get(name, 0.0) + a.elapsed_time(b)
            self.pending = []
        return self.ms

    def reset(self) -> None:
        self.collect()
        self.ms = {}


def install(timer) -> None:
    """Install a PhaseTimer (or None to switch profiling off)."""
    global _timer
    _timer = timer


def active():
    return _timer


def phase(name: str):
    return _NULL if _timer is None else _Span(_timer, name)
