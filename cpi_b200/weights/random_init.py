"""Random-weights mode: a model from a configuration and a seed, in memory or as a model folder.

The reference has no such mode (its substitute for real weights is the .ll2c
packing tool chain, tools/pack_ll2c.py).  Every tensor the model's parts declare
is drawn from N(0, initializer_range) in float32 and rounded to bfloat16, norm
weights are 1.  Each tensor has a generator of its own, seeded from (seed, tensor
name), so the values do not depend on the order of creation.  Values drawn on
the CPU and on a GPU differ (the two generators are different algorithms); a
model folder is always written from CPU draws.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .safetensors_io import write_safetensors
from .store import TensorReq, WeightSource


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


class RandomSource(WeightSource):
    """Draws each required tensor when it is asked for (nothing is held between calls)."""

    def __init__(self, reqs: list, seed: int, std: float, dtype: torch.dtype = torch.bfloat16):
        self.reqs = {}
        for r in reqs:
            if not r.optional:
                self.reqs[r.name] = r
        self.seed, self.std, self.dtype = int(seed), float(std), dtype

    def names(self):
        return list(self.reqs)

    def has(self, name):
        return name in self.reqs

    def shape(self, name):
        return tuple(self.reqs[name].shape)

    def stored_dtype(self, name):
        return self.dtype

    def get(self, name, device):
        r = self.reqs[name]
        device = torch.device(device)
        if r.init == "ones":
            return torch.ones(r.shape, dtype=self.dtype, device=device)
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(self.seed, name))
        if device.type == "cpu":
            t = torch.empty(r.shape, dtype=torch.float32).normal_(0.0, self.std, generator=g)
            return t.to(self.dtype)
        out = torch.empty(r.shape, dtype=self.dtype, device=device)
        flat = out.view(-1)
        step = 1 << 28                     # bound the float32 staging buffer
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.empty(n, dtype=torch.float32, device=device).normal_(
                0.0, self.std, generator=g).to(self.dtype)
        return out


def write_random_model(model_dir: str, config_json: dict, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Write `config.json` and `model.safetensors` for the architecture that config_json names."""
    from ..config.registry import architecture_of
    from ..engine.model import tensor_requirements
    arch = architecture_of(config_json)
    cfg = arch.parse_config(config_json)
    spec = arch.build_spec(cfg)
    spec.validate()
    reqs = tensor_requirements(spec)
    src = RandomSource(reqs, seed, spec.initializer_range, dtype)
    tensors = {name: src.get(name, "cpu") for name in src.names()}
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
