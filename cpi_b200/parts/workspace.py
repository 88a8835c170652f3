"""Named device buffers that live across steps, so that a step allocates nothing once it is warm."""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self._buffers: dict = {}
        self.generation = 0        # grows whenever a buffer is (re)allocated: captured graphs then hold stale addresses

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            cap = max(n, 1)
            if buf is not None:
                cap = max(cap, int(buf.numel() * 1.5))
            buf = torch.empty(cap, dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:n].view(*shape)

