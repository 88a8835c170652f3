"""safetensors container: read through mmap by tensor name, and write.

File format: 8-byte little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}`,
then the payload.  The reference maps every `*.safetensors` of a folder sorted
by file name and keeps only `data_offsets` (dtype and shape are skipped; first
occurrence of a name wins): src/model/safetensors_loader.cpp:305-376.  This
reader keeps dtype and shape as well, so that every tensor can be checked.
"""
from __future__ import annotations

import difflib
import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch


def nearest_name(name: str, names) -> str:
    """The name among `names` that most resembles `name`, or '' if nothing is close.  A wrong prefix is the
    usual mistake, so the longest shared tail of dotted components decides first, if it singles out one name."""
    names = [n for n in names if n != name]
    parts = name.split(".")
    for k in range(len(parts) - 1, 1, -1):
        tail = ".".join(parts[-k:])
        hits = [n for n in names if n == tail or n.endswith("." + tail)]
        if hits:
            if len(hits) == 1:
                return hits[0]
            break
    close = difflib.get_close_matches(name, names, n=1, cutoff=0.8)
    return close[0] if close else ""


class SafetensorsError(RuntimeError):
    pass


_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    shard: int
    begin: int      # absolute byte offset in the shard file
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


class SafetensorsDir:
    """All `*.safetensors` shards of a folder, indexed by tensor name."""

    def __init__(self, model_dir: str):
        if not os.path.isdir(model_dir):
            raise SafetensorsError(f"safetensors: not a folder: {model_dir}")
        files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
        if not files:
            raise SafetensorsError(f"safetensors: no *.safetensors file in {model_dir}")
        self.paths = [os.path.join(model_dir, f) for f in files]
        self._files = []
        self._maps = []
        self.entries: dict[str, TensorEntry] = {}
        for shard, path in enumerate(self.paths):
            f = open(path, "rb")
            self._files.append(f)
            size = os.fstat(f.fileno()).st_size
            if size < 8:
                raise SafetensorsError(f"safetensors: {path}: shorter than its 8-byte header length")
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps.append(m)
            (hlen,) = struct.unpack("<Q", m[:8])
            if 8 + hlen > size:
                raise SafetensorsError(f"safetensors: {path}: header length {hlen} exceeds file size {size}")
            try:
                header = json.loads(m[8:8 + hlen].decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"safetensors: {path}: header is not valid JSON ({e})") from None
            payload = 8 + hlen
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                if name in self.entries:      # first occurrence wins, as in the reference (:368-370)
                    continue
                try:
                    dt, shape, (b, e) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
                except (KeyError, TypeError, ValueError):
                    raise SafetensorsError(f"safetensors: {path}: malformed entry for '{name}'") from None
                if dt not in _DTYPES:
                    raise SafetensorsError(f"safetensors: {path}: tensor '{name}' has unsupported dtype {dt}")
                tdt, isz = _DTYPES[dt]
                n = 1
                for s in shape:
                    n *= int(s)
                if e < b or payload + e > size:
                    raise SafetensorsError(f"safetensors: {path}: tensor '{name}' data_offsets [{b}, {e}) "
                                           f"reach beyond the payload ({size - payload} bytes): truncated file?")
                if e - b != n * isz:
                    raise SafetensorsError(f"safetensors: {path}: tensor '{name}' has {e - b} bytes but "
                                           f"shape {list(shape)} of {dt} needs {n * isz}")
                self.entries[name] = TensorEntry(name, tdt, shape, shard, payload + b, payload + e)

    def names(self):
        return list(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def entry(self, name: str) -> TensorEntry:
        if name not in self.entries:
            near = nearest_name(name, self.entries)
            raise SafetensorsError(f"safetensors: tensor not found: {name}" + (f" (did you mean {near}?)" if near else ""))
        return self.entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (no copy); treat it as read-only."""
        e = self.entry(name)
        if e.nbytes == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = np.frombuffer(self._maps[e.shard], dtype=np.uint8, count=e.nbytes, offset=e.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # non-writable buffer
            t = torch.frombuffer(buf, dtype=torch.uint8)
        return t.view(e.dtype).view(e.shape)

    def close(self) -> None:
        for m in self._maps:
            try:
                m.close()
            except BufferError:
                pass
        for f in self._files:
            f.close()
        self._maps, self._files = [], []


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names; offsets are 8-byte aligned via header padding."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"safetensors: cannot write dtype {t.dtype} of '{name}'")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
