"""Architecture-independent description of a decoder: which parts each layer is made of.

An architecture (cpi_b200/models/*) turns its typed configuration into a
`ModelSpec`.  Everything below the spec -- parts, cache, engine, kernels -- sees
only these records, never a model name.  A part's sizes and constants travel in
its `params` dictionary; the part class registered under `kind` interprets them.

The reference has a single layer kind with its constants compiled in
(src/engine/llama4_cpu_engine.cpp:293-333); a spec with per-layer kinds and a
run order that is itself data has no counterpart there.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry key `kind` and the part's own parameters."""
    kind: str
    params: dict = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """A layer = a block arrangement of a mixer and a feed-forward with their norms.

    `prefix` is the tensor-name prefix under which the layer's weights live in the
    checkpoint; each part adds its own local names to it.
    """
    prefix: str
    block: PartSpec          # arrangement, e.g. kind "pre_norm"
    mixer: PartSpec          # e.g. kind "attention"
    feed_forward: PartSpec   # e.g. kind "dense_swiglu" or "moe_swiglu"
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    `layer` indexes `ModelSpec.layers`; a layer may be named by several entries
    (its weights are then used more than once).  `cache_of` is None when the
    entry keeps a cache / state of its own, or the index of an EARLIER run entry
    whose cache this entry reads without writing to it.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec            # kind "token_embedding", params: weight name
    layers: tuple                  # of LayerSpec
    run_order: tuple               # of RunEntry
    final_norm: PartSpec
    head: PartSpec                 # kind "linear_head", params: weight name (may alias the embedding)
    ignored_tensor_prefixes: tuple = ()
    bos_token_id: Optional[int] = None
    stop_token_ids: tuple = ()
    max_position: int = 0
    initializer_range: float = 0.02

    def validate(self) -> None:
        if not self.run_order:
            raise ValueError("ModelSpec.run_order is empty")
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run_order[{i}] names layer {e.layer} of {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"run_order[{i}].cache_of must name an earlier entry, got {e.cache_of}")
                if self.run_order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run_order[{i}].cache_of names entry {e.cache_of}, which itself "
                                     "reads another entry's cache")
                a = self.layers[e.layer].mixer
                b = self.layers[self.run_order[e.cache_of].layer].mixer
                if a.kind != b.kind:
                    raise ValueError(f"run_order[{i}] ({a.kind}) cannot read the cache of entry "
                                     f"{e.cache_of} ({b.kind})")
