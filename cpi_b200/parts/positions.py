"""Position encodings a mixer can apply to q and k.

"rope": rotary encoding with per-pair frequencies theta_d = theta^(-2d/D), optionally rescaled by the
llama3 rule; frequencies are computed on the host in float32 exactly as the reference does
(src/engine/llama4_cpu_engine.cpp:446-464), the angle float(p) * theta_d and its sine and cosine on
the device (the reference tabulates them, :466-470).  "none": q and k are used as projected.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Position, RotaryEncoding, register_position


def llama3_frequencies(head_dim: int, theta: float, scaling) -> np.ndarray:
    f32 = np.float32
    half = head_dim // 2
    out = np.empty(half, dtype=np.float32)
    for d in range(half):
        expo = f32(-2.0) * f32(d) / f32(head_dim)
        t = f32(np.power(f32(theta), expo, dtype=np.float32))
        if scaling is not None:
            orig = f32(scaling["original_max_position_embeddings"])
            low, high = f32(scaling["low_freq_factor"]), f32(scaling["high_freq_factor"])
            factor = f32(scaling["factor"])
            wavelen = f32(2.0) * f32(3.14159265358979323846) / t
            if wavelen > orig / low:
                t = t / factor
            elif wavelen >= orig / high:
                smooth = (orig / wavelen - low) / (high - low)
                t = (f32(1.0) - smooth) * (t / factor) + smooth * t
        out[d] = t
    return out


@register_position("rope")
class RotaryPosition(Position):
    """params: head_dim, theta, pairing ("half_split" pairs (d, d+D/2); "interleaved" pairs (2d, 2d+1)),
    scaling (None or the llama3 dictionary)."""
    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        sc = spec.get("scaling")
        if sc is not None and sc.get("rope_type", "llama3") != "llama3":
            raise ValueError(f"rope scaling of type '{sc.get('rope_type')}' is not supported")
        if spec["pairing"] not in ("half_split", "interleaved"):
            raise ValueError(f"unknown rope pairing '{spec['pairing']}'")
        self.interleaved = spec["pairing"] == "interleaved"
        self.frequencies = llama3_frequencies(int(spec["head_dim"]), float(spec["theta"]), sc)
        self.inv_freq = None

    def prepare(self, device):
        self.inv_freq = torch.from_numpy(self.frequencies).to(device)

    def encoding(self):
        return RotaryEncoding(self.inv_freq, self.interleaved)


@register_position("none")
class NoPosition(Position):
    graph_safe = True
