"""The engine: a loaded model, its cache, and ONE step function.

`step` takes, for each sequence of the batch, its slot, its next tokens and the places among them
whose logits are wanted.  The sequences of a batch start together (all at position 0, with unequal
prompt lengths, in one step) and then go on by one token each; a step runs only the tokens it is
given, against the cache that earlier steps left, as one packed batch without padding.  The
reference's counterpart is `forward_token(token, position)` for one sequence
(include/engine/llama4_cuda_engine.hpp:108-116); its "prefill" is a host loop over it
(src/engine/llama4_cuda_engine.cu:571-580).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..cache import CacheManager
from ..config.registry import apply_overrides, architecture_of, spec_from_model_dir
from ..config.spec import ModelSpec
from ..csrc import lib as K
from ..parts import Workspace
from .. import phases
from ..weights import RandomSource, SafetensorsSource
from .batch import BatchStager
from .model import DecoderModel


def _dtype_of(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if name not in table:
        raise ValueError(f"dtype must be bfloat16 or float32, not '{name}'")
    return table[name]


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Engine:
    def __init__(self, spec: ModelSpec, source, *, dtype="bfloat16", device="cuda:0", max_tokens: int = 4096,
                 max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None, page_size: int = 64,
                 max_step_tokens: int = 8192, config=None):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("cpi_b200 runs on a CUDA device only; there is no CPU path")
        K.load()                                   # fails loudly when the kernel library is missing
        torch.cuda.set_device(self.device)
        self.dtype = _dtype_of(dtype)
        self.spec, self.config = spec, config
        self.ws = Workspace(self.device)
        self.model = DecoderModel(spec, self.dtype, self.device, self.ws)
        self.model.load(source)
        kv, state = self.model.cache_requirements()
        self.max_step_tokens = max(1, int(max_step_tokens))
        self.cache = CacheManager(kv, state, max_tokens=max_tokens, max_seqs=max_seqs, max_seq_len=max_seq_len,
                                  page_size=page_size, dtype=self.dtype, device=self.device,
                                  max_step_tokens=self.max_step_tokens)
        self.stager = BatchStager(self.device)
        self.steps_run = 0
        # Decode steps (one token per sequence) are captured into CUDA graphs, one per (sequences, wanted
        # rows, context bucket): the first step of a kind runs eagerly, the second is captured, later ones
        # replay.  What changes from step to step -- tokens, positions, slots, page tables -- lives in
        # device buffers with fixed addresses that are refilled before each replay.  Only if every part of the
        # model declares itself safe for that (`Part.graph_safe`): a part that looks at host values of a step
        # would be replayed with those of the step that was captured.
        self.use_graphs = all(getattr(part, "graph_safe", False) for part in self.model.all_parts())
        self._graphs = {}
        self.graph_kernel_launches = 0       # kernels run by graph replays (they are not host launches)
        self._routing_capture = False
        self._phase_timer = None
        # What kernels flag on the device (a tensor-core kernel that gave up a wait, a token outside the
        # vocabulary) is copied to the host after every step, without waiting for it; the copy is looked at
        # when a later step starts and whenever the caller has synchronised anyway (`check_device_errors`).
        self._err_dev = K.device_error_flags(self.device)
        self._err_host = torch.zeros(2, dtype=torch.int32, pin_memory=True)
        self._err_event = None

    # ---- construction ----------------------------------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, config_overrides: Optional[dict] = None, **kw) -> "Engine":
        """`config_overrides`: config.json keys that replace the file's (for instance {"rope_theta": 1e6})."""
        cfg, spec = spec_from_model_dir(model_dir, config_overrides)
        src = SafetensorsSource(model_dir)
        try:
            return cls(spec, src, config=cfg, **kw)
        finally:
            src.close()

    @classmethod
    def from_random(cls, config_json: dict, seed: int = 0, config_overrides: Optional[dict] = None, **kw) -> "Engine":
        """A model with random weights drawn on the device (nothing is written to disk)."""
        from .model import tensor_requirements
        config_json = apply_overrides(config_json, config_overrides)
        arch = architecture_of(config_json)
        cfg = arch.parse_config(config_json)
        spec = arch.build_spec(cfg)
        src = RandomSource(tensor_requirements(spec), seed, spec.initializer_range)
        return cls(spec, src, config=cfg, **kw)

    # ---- slots -----------------------------------------------------------------------------------
    def acquire_slot(self) -> int:
        return self.cache.acquire()

    def release_slot(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    # ---- the step --------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the entries' tokens as one batch; returns float32 logits [wanted, vocab] on the device,
        in the order of the entries and of each entry's `want`."""
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        V = self.spec.vocab_size
        slots, toks, wants = [], [], []
        for e in entries:
            t = [int(x) for x in e.tokens]
            if not t:
                raise ValueError(f"slot {e.slot}: a step entry without tokens")
            for x in t:
                if not 0 <= x < V:
                    raise ValueError(f"slot {e.slot}: token id {x} is outside the vocabulary of {V}")
            w = [int(i) for i in e.want]
            for i in w:
                if not 0 <= i < len(t):
                    raise ValueError(f"slot {e.slot}: wanted place {i} is outside the entry's {len(t)} tokens")
            slots.append(int(e.slot)); toks.append(t); wants.append(w)
        n_new = [len(t) for t in toks]
        if sum(n_new) <= self.max_step_tokens:
            return self._run(slots, toks, wants)
        # A step larger than the workspace allows runs as pieces, one after the other: whole sequences
        # while they fit, and a longer sequence in runs of consecutive tokens.  Each piece attends to
        # what the pieces before it left in the cache, so the result is that of the single step.
        if len(set(slots)) != len(slots):
            raise ValueError("a step names the same slot twice")
        pieces, cur, cur_n = [], [], 0
        for s, t, w in zip(slots, toks, wants):
            off = 0
            while off < len(t):
                room = self.max_step_tokens - cur_n
                if room == 0:
                    pieces.append(cur)
                    cur, cur_n, room = [], 0, self.max_step_tokens
                n = min(room, len(t) - off)
                cur.append((s, t[off:off + n], [i - off for i in w if off <= i < off + n]))
                cur_n += n
                off += n
        if cur:
            pieces.append(cur)
        if any(sorted(w) != w for w in wants):
            raise ValueError("a step larger than max_step_tokens needs each entry's `want` in ascending order")
        # all pieces together must fit before the first one runs: a step is run whole or not at all
        self.cache.check_room([([c[0] for c in piece], [len(c[1]) for c in piece]) for piece in pieces])
        outs = [self._run([c[0] for c in piece], [c[1] for c in piece], [c[2] for c in piece]).clone()
                for piece in pieces]
        return torch.cat(outs, dim=0)

    def step_decode(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One more token for each slot, the token ids taken from an int32 device tensor [len(slots)]
        (for instance the sampler's output of the step before, which the host has not read yet); logits of
        every slot's token.  Otherwise the same as `step` with one-token entries."""
        B = len(slots)
        if B == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        if tokens.dtype != torch.int32 or tokens.numel() != B or tokens.device != self.device:
            raise ValueError("step_decode: tokens must be an int32 tensor on the engine's device, one per slot")
        return self._run([int(x) for x in slots], [[0]] * B, [[0]] * B, device_tokens=tokens)

    def _run(self, slots, toks, wants, device_tokens=None) -> torch.Tensor:
        """Runs one piece; the returned logits live in a buffer that the next step overwrites."""
        n_new = [len(t) for t in toks]
        self._raise_if_flagged(wait=False)          # what the step before last left, if its copy has arrived
        starts = self.cache.prepare_step(slots, n_new)
        decode = max(n_new) == 1
        if self._phase_timer is not None:
            self._phase_timer.kind = "decode" if decode else "prefill"
        if decode and self.use_graphs and not self._routing_capture and self._phase_timer is None:
            logits = self._run_decode_graph(slots, starts, toks, wants, device_tokens)
        else:
            batch = self.stager.stage(slots, starts, toks, wants, self.dtype)
            if device_tokens is not None:
                batch.tokens.copy_(device_tokens.view(-1))
            logits = self.model.run(batch, self.cache)
        self.cache.commit_step(slots, n_new)
        self.steps_run += 1
        self._err_host.copy_(self._err_dev, non_blocking=True)
        self._err_event = torch.cuda.Event()
        self._err_event.record()
        return logits

    def _run_decode_graph(self, slots, starts, toks, wants, device_tokens=None) -> torch.Tensor:
        B = len(slots)
        R = sum(len(w) for w in wants)
        longest = max(s + 1 for s in starts)
        bucket = 256
        while bucket < longest:
            bucket *= 2
        key = (B, R, bucket)
        st = self._graphs.get(key)
        gen = (self.ws.generation, K.scratch_generation)
        if st is not None and st["graph"] is not None and st["gen"] != gen:
            st = None                       # a buffer moved since the capture: the graph holds stale addresses
        if st is None:
            # first step of this kind: eager (it also sizes every workspace buffer and sets kernel attributes)
            dev = torch.empty(self.stager.words_needed(B, B, R), dtype=torch.int32, device=self.device)
            self._graphs[key] = {"dev": dev, "graph": None, "logits": None, "gen": None, "kernels": 0}
            batch = self.stager.stage(slots, starts, toks, wants, self.dtype, static_dev=dev)
            if device_tokens is not None:
                batch.tokens.copy_(device_tokens.view(-1))
            return self.model.run(batch, self.cache)
        batch = self.stager.stage(slots, starts, toks, wants, self.dtype, static_dev=st["dev"])
        if device_tokens is not None:
            batch.tokens.copy_(device_tokens.view(-1))          # after the staged copy, before the replay
        if st["graph"] is None:
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            before = K.kernel_launches()
            with torch.cuda.graph(g):
                st["logits"] = self.model.run(batch, self.cache)
            st["kernels"] = K.kernel_launches() - before
            st["graph"] = g
            st["gen"] = (self.ws.generation, K.scratch_generation)
        st["graph"].replay()
        self.graph_kernel_launches += st["kernels"]
        return st["logits"]

    # ---- inspection ------------------------------------------------------------------------------
    def capture_routing(self, on: bool = True) -> dict:
        """Starts (or stops) recording the experts chosen in every step.  Returns {layer index: list}
        whose lists grow by one int32 tensor [tokens, k] per step while recording is on."""
        out = {}
        self._routing_capture = bool(on)          # recording copies tensors every step: not inside a graph
        for i, layer in enumerate(self.model.layers):
            ff = layer.feed_forward
            if hasattr(ff, "capture"):
                ff.capture = [] if on else None
                if on:
                    out[i] = ff.capture
        return out

    def profile_phases(self, on: bool = True):
        """Starts (or stops) per-phase device timing of every step (the reference's profile_decode_phases,
        include/engine/llama_engine.hpp:65-98).  While on, steps run eagerly on one stream.  Returns the
        timer; `timer.collect()` gives {"prefill" | "decode": {phase: milliseconds}} summed over the steps."""
        self._phase_timer = phases.PhaseTimer() if on else None
        phases.install(self._phase_timer)
        return self._phase_timer

    def _raise_if_flagged(self, wait: bool) -> None:
        ev = self._err_event
        if ev is None or (not wait and not ev.query()):
            return
        ev.synchronize()
        self._err_event = None
        gave_up, token = int(self._err_host[0]), int(self._err_host[1])
        if not (gave_up or token):
            return
        self._err_dev.zero_()
        self._err_host.zero_()
        if gave_up:
            raise RuntimeError("a tensor-core kernel gave up waiting on one of its barriers; the results of the "
                               "steps since the last check are invalid")
        raise RuntimeError(f"embedding: token {token - 1} of a step was outside the vocabulary")

    def check_device_errors(self) -> None:
        """Raises if a kernel flagged a bad input or gave up a wait since the last check.  Waits for the device:
        `generate`, `Model.step` and the command lines call it where they have the results on the host anyway;
        between such points every step looks at what the step before it left, without waiting."""
        self._err_host.copy_(self._err_dev, non_blocking=True)
        self._err_event = torch.cuda.Event()
        self._err_event.record()
        self._raise_if_flagged(wait=True)
