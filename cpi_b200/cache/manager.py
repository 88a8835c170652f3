"""The cache: a slot per live sequence, paged keys and values per layer group, fixed-size state.

The reference holds one sequence in flat arrays [layer, max_ctx, kv] that are zeroed before every
generation (src/engine/llama4_cuda_engine_setup.cu:131-135, :456-465; indexing
src/engine/llama4_cuda_engine.cu:258-265).  Here:

* A **slot** stands for one live sequence: its length and, per group, its row of the page table.
  Slots come from a free list, go back when the sequence ends, and are used again.
* What a mixer keeps per position lives in **pages** of `page_size` positions.  Run entries whose mixers
  declare equal needs (same streams, same window) form a **group** with storage, page table and free
  list of its own.  A group stores one tensor per **stream** that its requirement names:
  `[entries, pages, heads, page_size, dim]`; attention's two streams are "k" and "v" of equal shape, a
  mixer that keeps something else per position (one compressed vector, say) names its own streams with
  their own shapes.  A sequence's block b (positions b*page_size ...) is page `table[slot, b]` of its
  group, for every stream alike.  Positions at or beyond a sequence's length are never read.
* A group with a window gives back, at the start of a step, the blocks that no later position can
  see (all positions before the chunk that holds the sequence's next position, or before the last
  `size` positions).
* **State**: a mixer may declare named tensors of fixed shape per sequence; they are kept as
  `[slots, *shape]` per run entry and zeroed when a slot is acquired.

All bookkeeping is on the host; tables are mirrored to the device before a step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot or no free page."""


@dataclass(frozen=True)
class KVRequirement:
    """What a mixer keeps per position.  By default two streams, "k" and "v", of `n_kv_heads` heads of
    `head_dim` elements; `streams` names others instead: a tuple of (name, heads, dim)."""
    n_kv_heads: int
    head_dim: int
    window_kind: str = "full"       # "full" | "chunk" | "sliding"
    window_size: int = 0
    streams: tuple = ()             # () = (("k", n_kv_heads, head_dim), ("v", n_kv_heads, head_dim))

    def stream_shapes(self) -> tuple:
        return self.streams or (("k", self.n_kv_heads, self.head_dim), ("v", self.n_kv_heads, self.head_dim))

    def first_needed_position(self, next_pos: int) -> int:
        """Smallest position that a query at `next_pos` or later can still see."""
        if self.window_kind == "chunk":
            return (next_pos // self.window_size) * self.window_size
        if self.window_kind == "sliding":
            return max(0, next_pos - self.window_size + 1)
        return 0


@dataclass(frozen=True)
class StateRequirement:
    """A named fixed-size tensor per sequence (shape without the slot axis)."""
    name: str
    shape: tuple
    dtype: torch.dtype = torch.float32


class PagePool:
    """Free list of page numbers with checks against double frees and leaks."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free page left (the group holds {self.n_pages})")
        p = self._free.pop()
        assert not self._held[p]
        self._held[p] = True
        return p

    def give_back(self, p: int) -> None:
        if not (0 <= p < self.n_pages) or not self._held[p]:
            raise CacheError(f"page {p} is given back but is not held")
        self._held[p] = False
        self._free.append(p)


class KVGroup:
    def __init__(self, req: KVRequirement, entries: list, n_pages: int, page_size: int, max_slots: int,
                 max_blocks: int, dtype: torch.dtype, device):
        self.req, self.entries = req, list(entries)
        self.page_size, self.max_blocks = page_size, max_blocks
        self.pool = PagePool(n_pages)
        # zeroed once: a tensor-core kernel multiplies masked positions by zero, which needs finite values
        self.streams = {}
        for name, heads, dim in req.stream_shapes():
            if name in self.streams:
                raise CacheError(f"a cache requirement names the stream '{name}' twice")
            self.streams[name] = torch.zeros((len(entries), n_pages, int(heads), page_size, int(dim)), dtype=dtype,
                                             device=device)
        self.k, self.v = self.streams.get("k"), self.streams.get("v")
        self.table_host = torch.zeros((max_slots, max_blocks), dtype=torch.int32)
        self.table = torch.zeros((max_slots, max_blocks), dtype=torch.int32, device=device)
        self.blocks: list[dict] = [dict() for _ in range(max_slots)]     # slot -> {block: page}
        self._dirty: set = set()
        self._index = {e: i for i, e in enumerate(self.entries)}

    def layer_views(self, entry: int):
        if self.k is None or self.v is None:
            raise CacheError(f"run entry {entry} keeps the streams {sorted(self.streams)}, not keys and values")
        i = self._index[entry]
        return self.k[i], self.v[i]

    def stream_view(self, entry: int, name: str):
        if name not in self.streams:
            raise CacheError(f"run entry {entry} keeps the streams {sorted(self.streams)}, not '{name}'")
        return self.streams[name][self._index[entry]]

    def ensure(self, slot: int, length: int, n_new: int) -> None:
        """Free what the window no longer needs, then hold a page for every block of [length, length+n_new)."""
        held = self.blocks[slot]
        first = self.req.first_needed_position(length) // self.page_size
        for b in [b for b in held if b < first]:
            self.pool.give_back(held.pop(b))
        if n_new <= 0:
            return
        last = (length + n_new - 1) // self.page_size
        if last >= self.max_blocks:
            raise CacheError(f"a sequence of {length + n_new} positions exceeds the cache's "
                             f"{self.max_blocks * self.page_size} positions per sequence")
        for b in range(length // self.page_size, last + 1):
            if b not in held:
                p = self.pool.take()
                held[b] = p
                self.table_host[slot, b] = p
                self._dirty.add(slot)

    def release(self, slot: int) -> None:
        held = self.blocks[slot]
        for b in list(held):
            self.pool.give_back(held.pop(b))

    def sync_tables(self) -> None:
        if not self._dirty:
            return
        if len(self._dirty) * 4 >= self.table_host.shape[0]:
            self.table.copy_(self.table_host, non_blocking=True)
        else:
            for s in sorted(self._dirty):
                self.table[s].copy_(self.table_host[s], non_blocking=True)
        self._dirty.clear()

    def pages_held(self) -> int:
        return sum(len(b) for b in self.blocks)


class CacheManager:
    """Slots, groups and state for one model on one device.

    `kv_requirements` / `state_requirements`: run-entry index -> requirement(s), only for entries that
    keep a cache of their own.  `max_tokens` bounds the positions all live sequences hold together,
    each sequence rounded up to whole pages; `max_seqs` the number of live sequences; `max_seq_len` the
    longest single sequence.
    """

    def __init__(self, kv_requirements: dict, state_requirements: dict, *, max_tokens: int,
                 max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None, page_size: int = 64,
                 dtype: torch.dtype = torch.bfloat16, device="cuda", max_step_tokens: Optional[int] = None):
        if page_size < 1 or max_tokens < 1:
            raise CacheError("page_size and max_tokens must be positive")
        self.page_size = page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_slots = max_seqs if max_seqs is not None else self.n_pages
        self.max_seq_len = max_seq_len if max_seq_len is not None else self.n_pages * page_size
        self.max_blocks = -(-self.max_seq_len // page_size)
        self.device, self.dtype = device, dtype
        by_req: dict = {}
        for entry, req in sorted(kv_requirements.items()):
            by_req.setdefault(req, []).append(entry)
        # A group with a window never holds more of a sequence than the window and the step that is being
        # added (pages before the window are given back when a step starts), so its storage is sized for
        # that and not for whole sequences: `max_step_tokens` is the most tokens one step brings a sequence.
        self.max_step_tokens = max_step_tokens
        self.groups = [KVGroup(req, entries, self.pages_for(req), page_size, self.max_slots, self.max_blocks,
                               dtype, device) for req, entries in by_req.items()]
        self.group_of_entry = {e: g for g in self.groups for e in g.entries}
        self.state: dict = {}
        for entry, reqs in sorted(state_requirements.items()):
            for r in reqs:
                self.state[(entry, r.name)] = torch.zeros((self.max_slots, *r.shape), dtype=r.dtype,
                                                          device=device)
        self._free_slots = list(range(self.max_slots - 1, -1, -1))
        self._live = [False] * self.max_slots
        self.lengths = [0] * self.max_slots

    def pages_for(self, req: KVRequirement) -> int:
        """Pages that a group of this requirement gets: all of the cache's for full attention; for a window,
        per sequence the window plus one step, if that is less."""
        if req.window_kind == "full" or self.max_step_tokens is None or req.window_size <= 0:
            return self.n_pages
        span = min(self.max_seq_len, req.window_size - 1 + min(self.max_step_tokens, self.max_seq_len))
        per_seq = -(-span // self.page_size) + 1          # a span that starts inside a page touches one page more
        return max(1, min(self.n_pages, self.max_slots * per_seq))

    # ---- slots ---------------------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def live_slots(self) -> list:
        return [s for s in range(self.max_slots) if self._live[s]]

    def acquire(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.max_slots} sequence slots are in use")
        s = self._free_slots.pop()
        assert not self._live[s]
        self._live[s] = True
        self.lengths[s] = 0
        for t in self.state.values():
            t[s].zero_()
        return s

    def release(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots) or not self._live[slot]:
            raise CacheError(f"slot {slot} is released but is not live")
        for g in self.groups:
            g.release(slot)
        self._live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    # ---- steps ---------------------------------------------------------------------------------
    def check_room(self, pieces: list) -> None:
        """Raises, having changed nothing, unless the cache can hold what `pieces` bring: a list of
        (slots, n_new) that will run one after the other (a single step is one piece).  Per group the pages
        are counted as the steps would take and give them back, windows included, in the same order."""
        ps = self.page_size
        lengths: dict = {}
        for slots, n_new in pieces:
            if len(set(slots)) != len(slots):
                raise CacheError("a step names the same slot twice")
            for s, n in zip(slots, n_new):
                if not (0 <= s < self.max_slots) or not self._live[s]:
                    raise CacheError(f"slot {s} is stepped but is not live")
                if n < 1:
                    raise CacheError(f"slot {s}: a step must bring at least one token")
                at = lengths.get(s, self.lengths[s])
                if at + n > self.max_seq_len:
                    raise CacheError(f"slot {s}: {at} + {n} positions exceed the longest sequence the cache "
                                     f"was sized for ({self.max_seq_len})")
                lengths[s] = at + n
        for g in self.groups:
            free = g.pool.free_count
            held: dict = {}
            at: dict = {}
            for slots, n_new in pieces:
                for s, n in zip(slots, n_new):
                    h = held.setdefault(s, set(g.blocks[s]))
                    length = at.get(s, self.lengths[s])
                    first = g.req.first_needed_position(length) // ps
                    gone = {b for b in h if b < first}
                    free += len(gone)
                    h -= gone
                    for b in range(length // ps, (length + n - 1) // ps + 1):
                        if b not in h:
                            h.add(b)
                            free -= 1
                    if free < 0:
                        raise CacheFull(f"the cache is full: {self.tokens_held()} of {self.n_pages * ps} "
                                        f"positions are held by {len(self.live_slots())} sequences and the step "
                                        f"needs more than the rest (group with window '{g.req.window_kind}': "
                                        f"{g.pool.n_pages} pages)")
                    at[s] = length + n

    def prepare_step(self, slots: list, n_new: list) -> list:
        """Hold pages for the new positions of each sequence; returns the start position of each.  Either
        every sequence of the step gets its pages or nothing changes."""
        self.check_room([(slots, n_new)])
        starts = [self.lengths[s] for s in slots]
        for s, n in zip(slots, n_new):
            for g in self.groups:
                g.ensure(s, self.lengths[s], n)
        for g in self.groups:
            g.sync_tables()
        return starts

    def commit_step(self, slots: list, n_new: list) -> None:
        for s, n in zip(slots, n_new):
            self.lengths[s] += n

    # ---- views ---------------------------------------------------------------------------------
    def kv_view(self, entry: int):
        """(k, v, page_table, page_size) of the group that holds run entry `entry`."""
        g = self.group_of_entry[entry]
        k, v = g.layer_views(entry)
        return k, v, g.table, g.page_size

    def stream_view(self, entry: int, name: str):
        """(tensor [pages, heads, page_size, dim], page_table, page_size) of one named stream of run entry `entry`."""
        g = self.group_of_entry[entry]
        return g.stream_view(entry, name), g.table, g.page_size

    def state_view(self, entry: int, name: str) -> torch.Tensor:
        return self.state[(entry, name)]

    def tokens_held(self) -> int:
        return max((g.pages_held() for g in self.groups), default=0) * self.page_size

    def check_consistency(self) -> None:
        """Every page is free or held by exactly one live slot; no slot is both free and live."""
        if sorted(self._free_slots + self.live_slots()) != list(range(self.max_slots)):
            raise CacheError("slot bookkeeping is inconsistent")
        for g in self.groups:
            held = [p for s, blocks in enumerate(g.blocks) for p in blocks.values()]
            if len(set(held)) != len(held):
                raise CacheError("a page is held twice")
            for s, blocks in enumerate(g.blocks):
                if blocks and not self._live[s]:
                    raise CacheError(f"free slot {s} still holds pages")
            if len(held) + g.pool.free_count != g.pool.n_pages:
                raise CacheError("pages were lost")
