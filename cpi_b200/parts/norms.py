"""RMS norm: y = x * rsqrt(mean(x^2) + eps) * w  (src/engine/llama4_cpu_engine.cpp:47-62)."""
from __future__ import annotations

from ..csrc import lib as K
from ..weights.store import TensorReq
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, weight (tensor name relative to the prefix, or None for a weightless norm)."""
    graph_safe = True

    def __init__(self, spec, prefix="", workspace=None, tag="norm"):
        super().__init__(spec, prefix)
        self.size, self.eps = int(spec["size"]), float(spec["eps"])
        self.weight_name = None if spec.get("weight") is None else prefix + spec["weight"]
        self.weight = None
        self.ws, self.tag = workspace, tag

    def requirements(self):
        if self.weight_name is None:
            return []
        return [TensorReq(self.weight_name, (self.size,), init="ones")]

    def load(self, source, device):
        if self.weight_name is not None:
            self.weight = source.get(self.weight_name, device).contiguous()

    def __call__(self, x, out_dtype, rows=None, out=None):
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = self.ws.get(self.tag, (n, self.size), out_dtype)
        K.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
