"""Weights by tensor name: what a model needs, what a source holds, and one error for every mismatch.

The reference fetches tensors by HF name (src/engine/llama4_cpu_engine.cpp:419-443),
checks byte sizes in its CUDA engine only ("unexpected tensor size for <name>",
src/engine/llama4_cuda_engine_setup.cu:223-227) and assumes bf16 throughout.  Here
the model's parts declare each tensor they need with its shape; `check_source`
compares that list with the source once and raises a single `WeightsError` that
lists missing tensors, unexpected tensors and wrong shapes together.

Storage dtypes: BF16 stays bfloat16; F32 stays float32; F16 is widened to float32
(exact); integer tensors become int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

import torch

from .safetensors_io import SafetensorsDir, nearest_name


class WeightsError(RuntimeError):
    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


@dataclass(frozen=True)
class TensorReq:
    """A tensor a part needs: full name, shape, how a random model fills it."""
    name: str
    shape: tuple
    init: str = "normal"        # "normal" (std = initializer range) or "ones"
    optional: bool = False      # absent is fine; the part asks `source.has(name)`


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    if stored == torch.bfloat16:
        return torch.bfloat16
    if stored in (torch.float32, torch.float16, torch.float64):
        return torch.float32
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    raise WeightsError(f"unsupported stored dtype {stored}")


class WeightSource:
    """Interface: tensors by name.  `get` returns the tensor in its kept dtype on `device`."""

    def names(self) -> Iterable[str]:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        raise NotImplementedError

    def shape(self, name: str) -> tuple:
        raise NotImplementedError

    def stored_dtype(self, name: str) -> torch.dtype:
        raise NotImplementedError

    def get(self, name: str, device) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass


class SafetensorsSource(WeightSource):
    def __init__(self, model_dir: str):
        self.dir = SafetensorsDir(model_dir)

    def names(self):
        return self.dir.names()

    def has(self, name):
        return name in self.dir

    def shape(self, name):
        return tuple(self.dir.entry(name).shape)

    def stored_dtype(self, name):
        return self.dir.entry(name).dtype

    def get(self, name, device):
        t = self.dir.tensor(name)
        kd = kept_dtype(t.dtype)
        if torch.device(device).type == "cpu":
            return t.to(kd).clone() if t.dtype == kd else t.to(kd)
        if t.dtype == torch.float16 and kd == torch.float32:
            # the stored bytes go up as they are and are widened on the device by the kernel library
            from ..csrc import lib as K
            raw = t.to(device=device, non_blocking=False).contiguous()
            out = torch.empty(raw.shape, dtype=torch.float32, device=device)
            K.widen_f16(raw, out)
            return out
        return t.to(device=device, dtype=kd, non_blocking=False)

    def close(self):
        self.dir.close()


class DictSource(WeightSource):
    """Tensors held in a dictionary (tests, and models built in memory)."""

    def __init__(self, tensors: dict):
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def has(self, name):
        return name in self.tensors

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def stored_dtype(self, name):
        return self.tensors[name].dtype

    def get(self, name, device):
        t = self.tensors[name]
        return t.to(device=device, dtype=kept_dtype(t.dtype))


def check_source(reqs: list, source: WeightSource, ignored_prefixes: tuple = (),
                 tolerated: tuple = ()) -> None:
    """Raise one WeightsError naming every missing / unexpected / mis-shaped tensor."""
    wanted = {}
    for r in reqs:
        if r.name in wanted and wanted[r.name].shape != tuple(r.shape):
            raise WeightsError(f"tensor '{r.name}' is required with two shapes: "
                               f"{list(wanted[r.name].shape)} and {list(r.shape)}")
        wanted[r.name] = r
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, r in wanted.items():
        if not source.has(name):
            if not r.optional:
                missing.append(name)
            continue
        got = tuple(source.shape(name))
        if got != tuple(r.shape):
            wrong_shape.append((name, tuple(r.shape), got))
        sd = source.stored_dtype(name)
        if not sd.is_floating_point:
            wrong_dtype.append((name, sd))
    unexpected = [n for n in source.names()
                  if n not in wanted and n not in tolerated
                  and not any(n.startswith(p) for p in ignored_prefixes)]
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = ["the weights do not match the model's configuration:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}):")
        for n in sorted(missing):
            near = nearest_name(n, unexpected)
            lines.append(f"    {n}  expected shape {list(wanted[n].shape)}" + (f"  (did you mean {near}?)" if near else ""))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}):")
        lines += [f"    {n}  shape {list(source.shape(n))}" for n in sorted(unexpected)]
    if wrong_shape:
        lines.append(f"  wrong shapes ({len(wrong_shape)}):")
        lines += [f"    {n}  expected {list(e)}, found {list(g)}" for n, e, g in sorted(wrong_shape)]
    if wrong_dtype:
        lines.append(f"  wrong dtypes ({len(wrong_dtype)}):")
        lines += [f"    {n}  stored as {d}, expected a floating-point type" for n, d in sorted(wrong_dtype)]
    raise WeightsError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)
