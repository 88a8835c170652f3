"""Random-weights mode: a model from a configuration and a seed, in memory or as a model folder.

The reference has no such mode (its substitute for real weights is the .ll2c
packing tool chain, tools/pack_ll2c.py).  Every tensor the model's parts declare
is drawn from N(0, initializer_range) and rounded to bfloat16, norm weights are 1.
The generator is counter based: element i of a tensor is a function of (seed,
tensor name, i) alone, computed with integer arithmetic, one table look-up and one
multiplication, so the values depend neither on the order of creation nor on the
device: a model drawn on a GPU equals the folder written from the CPU bit for bit.
"""
from __future__ import annotations

import hashlib
import json
import math
import os

import torch

from .safetensors_io import write_safetensors
from .store import WeightSource


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _i64(c: int) -> int:
    """A 64-bit constant as the signed integer that torch's int64 holds."""
    return c - (1 << 64) if c >= (1 << 63) else c


_TABLE = None


def _normal_table() -> torch.Tensor:
    """Inverse normal distribution function at the 65,536 bin centres (float32, computed once on the CPU in
    float64): a draw is one of these values, chosen by 16 hashed bits."""
    global _TABLE
    if _TABLE is None:
        u = (torch.arange(65536, dtype=torch.float64) + 0.5) / 65536.0
        _TABLE = (math.sqrt(2.0) * torch.erfinv(2.0 * u - 1.0)).to(torch.float32)
    return _TABLE


_TABLE_DEV: dict = {}


def _normal_table_on(device) -> torch.Tensor:
    key = str(device)
    if key not in _TABLE_DEV:
        _TABLE_DEV[key] = _normal_table().to(device).contiguous()
    return _TABLE_DEV[key]


def counter_normal(tensor_seed: int, start: int, n: int, std: float, device) -> torch.Tensor:
    """float32 [n]: the draws number start .. start + n - 1 of the stream `tensor_seed`.  Integer mixing
    (64-bit multiplications wrap and shifts are made logical by a mask: the same on every device), 16 bits
    pick the table entry."""
    i = torch.arange(start, start + n, dtype=torch.int64, device=device)
    z = i * _i64(0x9E3779B97F4A7C15) + tensor_seed
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _i64(0xBF58476D1CE4E5B9)
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _i64(0x94D049BB133111EB)
    z = z ^ ((z >> 31) & ((1 << 33) - 1))
    idx = (z >> 48) & 0xFFFF
    return _normal_table().to(device)[idx] * std


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
        ts = _tensor_seed(self.seed, name)
        out = torch.empty(r.shape, dtype=self.dtype, device=device)
        if device.type == "cuda" and self.dtype in (torch.bfloat16, torch.float32):
            # on a GPU the kernel library draws the tensor in place: the same integer arithmetic, the same bits
            from ..csrc import lib as K
            K.random_normal(out, 0, ts, self.std, _normal_table_on(device))
            return out
        flat = out.view(-1)
        step = 1 << 26                     # bound the int64 staging buffers
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = counter_normal(ts, i, n, self.std, device).to(self.dtype)
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
