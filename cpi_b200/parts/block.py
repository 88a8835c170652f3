"""Arrangement of a layer's parts.  "pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x))
(the order of src/engine/llama4_cpu_engine.cpp:300-329)."""
from __future__ import annotations

from ..phases import phase
from .base import Block, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    graph_safe = True
    def __init__(self, spec, prefix="", **_):
        super().__init__(spec, prefix)

    def run(self, layer, residual, batch, cache):
        with phase("rmsnorm"):
            h = layer.mixer_norm(residual, batch.dtype)
        layer.mixer.forward(h, residual, batch, cache)
        with phase("rmsnorm"):
            h2 = layer.feed_forward_norm(residual, batch.dtype)
        layer.feed_forward.forward(h2, residual, batch)
