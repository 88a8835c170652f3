"""What one step runs: the packed tokens of its sequences and where each token sits.

Every array is int32 on the device, filled from one pinned host buffer with a single copy:
  tokens[t]     token id                    token_seq[t]  index of its sequence in this step
  token_pos[t]  absolute position           seq_slot[s]   cache slot of sequence s
  seq_start[s]  positions cached before     seq_new[s]    tokens the step brings for s
  want_rows[r]  packed token indices whose logits are asked for
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


from ..csrc.lib import PREFILL_TILE_ROWS as Q_TILE      # query rows that one block of the prefill attention kernel takes


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    n_want: int
    max_new: int
    dtype: torch.dtype
    tokens: torch.Tensor
    token_seq: torch.Tensor
    token_pos: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_new: torch.Tensor
    want_rows: torch.Tensor
    slots: list
    starts: list
    n_new: list
    ctx_bucket: int = 0                # an upper bound of the longest context, a power of two (sizes key splits)
    n_q_tiles: int = 0                 # prefill only: tiles of up to Q_TILE consecutive tokens of one sequence,
    tile_tok0: torch.Tensor = None     # first packed token of each tile, longest context first
    tile_rows: torch.Tensor = None     # tokens in each tile

    @property
    def is_decode(self) -> bool:
        return self.max_new == 1


class BatchStager:
    """Builds StepBatch objects.  Index arrays go through a small ring of pinned host buffers, each
    with a device twin; a buffer is written again only after the copy that last read it has finished,
    so the host never waits for the step before last."""

    RING = 4

    def __init__(self, device):
        self.device = torch.device(device)
        self._cap = 0
        self._ring = []
        self._next = 0
        self.bytes_staged = 0          # host-to-device bytes of the latest step

    @staticmethod
    def words_needed(n_tokens: int, n_seqs: int, n_want: int) -> int:
        """int32 words a decode step (one token per sequence, no query tiles) stages."""
        return 3 * n_tokens + 3 * n_seqs + n_want

    def _reserve(self, n: int) -> None:
        if n <= self._cap:
            return
        self._cap = max(n, int(self._cap * 1.5), 4096)
        pin = self.device.type == "cuda"
        self._ring = []
        for _ in range(self.RING):
            host = torch.empty(self._cap, dtype=torch.int32, pin_memory=pin)
            dev = torch.empty(self._cap, dtype=torch.int32, device=self.device)
            self._ring.append([host, dev, None])

    def stage(self, slots, starts, token_lists, wants, dtype, static_dev=None) -> StepBatch:
        """`static_dev`: an int32 device buffer to fill instead of the ring's (its address then stays the
        same from step to step, which a captured CUDA graph needs)."""
        B = len(slots)
        n_new = [len(t) for t in token_lists]
        T = sum(n_new)
        R = sum(len(w) for w in wants)
        tiles = []
        if max(n_new) > 1:
            base = 0
            for n, st in zip(n_new, starts):
                for off in range(0, n, Q_TILE):
                    rows = min(Q_TILE, n - off)
                    tiles.append((st + off + rows, base + off, rows))
                base += n
            tiles.sort(key=lambda x: -x[0])          # most keys first: the long tiles start early
        total = 3 * T + 3 * B + R + 2 * len(tiles)
        self._reserve(total)
        entry = self._ring[self._next]
        self._next = (self._next + 1) % self.RING
        h, d, ev = entry
        if static_dev is not None:
            d = static_dev
        if ev is not None:
            ev.synchronize()
        tokens, token_seq, token_pos, want_rows = [], [], [], []
        base = 0
        for s, (toks, st, w) in enumerate(zip(token_lists, starts, wants)):
            n = len(toks)
            tokens += toks
            token_seq += [s] * n
            token_pos += range(st, st + n)
            want_rows += [base + i for i in w]
            base += n
        flat = (tokens + token_seq + token_pos + list(slots) + list(starts) + n_new + want_rows
                + [t[1] for t in tiles] + [t[2] for t in tiles])
        h[:total] = torch.tensor(flat, dtype=torch.int32)
        d[:total].copy_(h[:total], non_blocking=True)
        self.bytes_staged = total * 4
        if self.device.type == "cuda":
            entry[2] = torch.cuda.Event()
            entry[2].record()
        o = 0

        def take(n):
            nonlocal o
            v = d[o:o + n]
            o += n
            return v

        longest = max(st + n for st, n in zip(starts, n_new))
        bucket = 256
        while bucket < longest:
            bucket *= 2
        return StepBatch(n_tokens=T, n_seqs=B, n_want=R, max_new=max(n_new), dtype=dtype, ctx_bucket=bucket,
                         tokens=take(T), token_seq=take(T), token_pos=take(T), seq_slot=take(B),
                         seq_start=take(B), seq_new=take(B), want_rows=take(R),
                         slots=list(slots), starts=list(starts), n_new=n_new,
                         n_q_tiles=len(tiles), tile_tok0=take(len(tiles)), tile_rows=take(len(tiles)))
