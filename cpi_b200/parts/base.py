"""Interfaces of the parts a layer is put together from, and the registries that name them.

A part is built from a `PartSpec` (its kind and its own parameters) and a tensor-name prefix.  It
declares the tensors it needs, loads them (fusing or transposing as it likes), and runs on the tokens
of a step.  No part knows which model it is in: what it may use is its parameters, its weights, the
step's `StepBatch`, and -- for mixers -- the cache and state views the engine hands it.

Interfaces
----------
Norm          requirements(); load(src, dev); __call__(x, out_dtype, rows=None) -> tensor
Position      (no weights) prepare(dev); encoding() -> RotaryEncoding | ScoreBias | None, consumed by its mixer
Mixer         requirements(); load(src, dev); kv_requirement(); state_requirements();
              forward(h, residual, batch, cache)        # residual += mixer(h)
FeedForward   requirements(); load(src, dev); forward(h, residual, batch)   # residual += ffn(h)
Block         run(layer, residual, batch, cache)        # the arrangement of the above

`h` is the normed input in the activation dtype [tokens, hidden]; `residual` is the float32 residual
stream [tokens, hidden], updated in place.  A mixer must give the same result for a position whether
the sequence's tokens come in one step or one at a time; what it needs to remember lives in `cache`.

A new kind is added with `register_mixer("name")(cls)` (likewise for the others) and is then chosen
by a `PartSpec` of that kind; nothing else in the library changes.  A part whose step depends on the step
only through device buffers sets `graph_safe = True`; decode steps of a model are captured into CUDA
graphs only if all its parts do.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from ..config.spec import PartSpec


class Part:
    # Whether a decode step through this part may be captured into a CUDA graph and replayed: its launches
    # must then depend on the step only through device buffers (tokens, positions, slots, page tables),
    # never through host values such as `batch.slots`, data-dependent shapes or a synchronisation.  A part
    # says so itself; the default is no, and the engine replays graphs only if every part of the model does.
    graph_safe = False

    def __init__(self, spec: PartSpec, prefix: str = ""):
        self.spec, self.prefix = spec, prefix

    def requirements(self) -> list:
        return []

    def load(self, source, device) -> None:
        pass


class Norm(Part):
    def __call__(self, x, out_dtype, rows=None, out=None):
        raise NotImplementedError


@dataclass(frozen=True)
class RotaryEncoding:
    """q and k are rotated pairwise: the pair d of a head at position p turns by the angle p * inv_freq[d]
    (float32 [head_dim / 2] on the device); `interleaved` pairs (2d, 2d + 1), otherwise (d, d + head_dim / 2)."""
    inv_freq: torch.Tensor
    interleaved: bool = False


@dataclass(frozen=True)
class ScoreBias:
    """Positions act on the attention scores: table[head, min(query position - key position, n - 1)] (float32
    [heads, n] on the device) is added to the scaled score of a query and a key; q and k stay as projected."""
    table: torch.Tensor


class Position(Part):
    """How positions enter a mixer.  `prepare` builds device tables; `encoding()` then says what the part is to
    its mixer: a `RotaryEncoding`, a `ScoreBias`, or None (positions do not enter).  A mixer takes the kinds
    its kernels know and refuses the others by name."""

    def prepare(self, device) -> None:
        pass

    def encoding(self):
        return None


class Mixer(Part):
    """Built with `owns_cache=False` when every run entry of its layer reads another entry's cache."""

    def kv_requirement(self):
        return None

    def state_requirements(self) -> list:
        return []

    def forward(self, h, residual, batch, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, residual, batch) -> None:
        raise NotImplementedError


class Block(Part):
    def run(self, layer, residual, batch, cache) -> None:
        raise NotImplementedError


class CacheView:
    """What a mixer sees of the cache during one step, for its run entry."""

    def __init__(self, manager, entry: int, owns: bool = True):
        self._m, self._entry = manager, entry
        self.owns = owns          # False: this run entry reads `entry`'s cache and must not write it

    def kv(self):
        """(k, v, page_table, page_size): k, v are [pages, kv heads, page_size, head_dim]."""
        return self._m.kv_view(self._entry)

    def stream(self, name: str):
        """(tensor [pages, heads, page_size, dim], page_table, page_size) of a stream that the mixer's
        `KVRequirement.streams` names (attention's are "k" and "v")."""
        return self._m.stream_view(self._entry, name)

    def state(self, name: str) -> torch.Tensor:
        """[slots, *shape] tensor of the named per-sequence state."""
        return self._m.state_view(self._entry, name)


_REGISTRIES: dict = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}}


def _register(family: str, kind: str) -> Callable:
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        return cls
    return deco


def register_norm(kind): return _register("norm", kind)
def register_position(kind): return _register("position", kind)
def register_mixer(kind): return _register("mixer", kind)
def register_feed_forward(kind): return _register("feed_forward", kind)
def register_block(kind): return _register("block", kind)


def build_part(family: str, spec: PartSpec, prefix: str = "", **kw):
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise KeyError(f"no {family} of kind '{spec.kind}' is registered; registered: {sorted(reg)}")
    return reg[spec.kind](spec, prefix, **kw)


def registered(family: str) -> list:
    return sorted(_REGISTRIES[family])
