"""Trace replay: given token ids go through the engine step by step and the logits are written out.

Nothing is sampled.  A step is a JSON object
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
whose requests either all start at their first token or all go on by one token.  `TraceRunner.run` feeds it to
`Engine.step` -- the model, cache and kernels that generation uses -- and writes, for a step that wants
something, `<out>/<step>.f32`: little-endian float32 [wanted, vocab] in the order of the entries and of `want`;
with `dump_routing` also `<out>/<step>.routing.i32`: int32 [routed layers, tokens of the step, k], the experts
each token chose, in the order of the entries.  `index.json` (written by `close`) lists for every step its
entries with their start positions, so that a row of a file is a (request, position).

The three schedules that the parity tests replay are made here as lists of such steps from a trace file
(`id: t0 t1 t2 ...` per line): `whole` (each request alone, all tokens in one step, logits everywhere), `tail`
(each request alone, all but its last n tokens in one step, then one token per step) and `batched` (requests
in groups that start together with their prompts, then bring one token each per step; a shorter request ends
earlier; group follows group, so that slots and pages are used again).

The reference has no such tool; its nearest aids print the top-k logits after a prompt
(src/app/main_modes.cpp:275-285) or re-run the whole prompt for every greedy step (:286-313), over
`inspect_next_logits` (src/engine/llama4_cuda_engine.cu:623-674).
"""
from __future__ import annotations

import json
import os
from typing import Iterable, Iterator


def read_trace(path: str) -> dict:
    """{request id: [token ids]} of a trace file, in the file's order; one request per line, `id: t0 t1 ...`
    (blanks or commas between the ids; empty lines and lines that start with # are skipped)."""
    out: dict = {}
    with open(path, "r", encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            if ":" not in line:
                raise ValueError(f"{path}:{n}: expected 'id: t0 t1 ...'")
            rid, rest = line.split(":", 1)
            rid = rid.strip()
            toks = [int(x) for x in rest.replace(",", " ").split()]
            if not rid or not toks:
                raise ValueError(f"{path}:{n}: a request needs an id and at least one token")
            if rid in out:
                raise ValueError(f"{path}:{n}: request id '{rid}' appears twice")
            out[rid] = toks
    if not out:
        raise ValueError(f"{path}: no requests")
    return out


def schedule_whole(requests: dict) -> Iterator[dict]:
    for step, (rid, toks) in enumerate(requests.items()):
        yield {"step": step, "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
               "end": [rid]}


def schedule_tail(requests: dict, tail: int = 32) -> Iterator[dict]:
    """Logits at the last token of the first step and at every token after it."""
    step = 0
    for rid, toks in requests.items():
        n = len(toks)
        head = max(1, n - tail)
        yield {"step": step, "entries": [{"id": rid, "tokens": list(toks[:head]), "want": [head - 1]}],
               "end": [rid] if head == n else []}
        step += 1
        for i in range(head, n):
            yield {"step": step, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                   "end": [rid] if i == n - 1 else []}
            step += 1


def schedule_batched(requests: dict, batch_size: int, tail: int = 32) -> Iterator[dict]:
    """Groups of `batch_size` requests in the trace's order.  A request's prompt is all but its last `tail` tokens
    (at least one token); it ends with the step that brings its last token."""
    if batch_size < 1:
        raise ValueError("batch size must be >= 1")
    ids = list(requests)
    step = 0
    for b in range(0, len(ids), batch_size):
        group = ids[b:b + batch_size]
        head = {rid: max(1, len(requests[rid]) - tail) for rid in group}
        yield {"step": step,
               "entries": [{"id": rid, "tokens": list(requests[rid][:head[rid]]), "want": [head[rid] - 1]}
                           for rid in group],
               "end": [rid for rid in group if head[rid] == len(requests[rid])]}
        step += 1
        live = [rid for rid in group if head[rid] < len(requests[rid])]
        k = 0
        while live:
            yield {"step": step,
                   "entries": [{"id": rid, "tokens": [requests[rid][head[rid] + k]], "want": [0]} for rid in live],
                   "end": [rid for rid in live if head[rid] + k == len(requests[rid]) - 1]}
            step += 1
            k += 1
            live = [rid for rid in live if head[rid] + k < len(requests[rid])]


def tokens_needed(steps: Iterable[dict], page: int = 64) -> int:
    """The most tokens that live requests hold at any time in a schedule, each rounded up to `page`."""
    held: dict = {}
    most = 0
    for s in steps:
        for e in s.get("entries", []):
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-n // page) * page for n in held.values()))
        for rid in s.get("end", []):
            held.pop(rid, None)
    return most


class TraceRunner:
    """Feeds steps to an engine and writes what they want into `out_dir`."""

    def __init__(self, engine, out_dir: str, dump_routing: bool = False):
        from .engine import StepEntry
        self._entry = StepEntry
        self.engine, self.out_dir = engine, out_dir
        os.makedirs(out_dir, exist_ok=True)
        self.slots: dict = {}
        self.index: list = []
        self._routing = engine.capture_routing(True) if dump_routing else None
        self._top_k = 0

    def run(self, obj: dict) -> None:
        import torch
        eng = self.engine
        step = obj["step"]
        entries, layout = [], []
        for e in obj.get("entries", []):
            rid = str(e["id"])
            if rid not in self.slots:
                self.slots[rid] = eng.acquire_slot()
            slot = self.slots[rid]
            want = [int(w) for w in e.get("want", [])]
            layout.append({"id": rid, "start": eng.length(slot), "tokens": len(e["tokens"]), "want": want})
            entries.append(self._entry(slot, e["tokens"], want))
        if self._routing is not None:
            for lst in self._routing.values():
                lst.clear()
        record = {"step": step, "file": None, "routing": None, "entries": layout}
        if entries:
            logits = eng.step(entries)
            if logits.shape[0] > 0:
                record["file"] = f"{step}.f32"
                logits.detach().cpu().numpy().astype("<f4", copy=False).tofile(os.path.join(self.out_dir, record["file"]))
            else:
                torch.cuda.synchronize(eng.device)
            if self._routing:
                # a step that ran as pieces recorded one tensor per piece, in the packed order of the step
                layers = sorted(self._routing)
                chosen = torch.stack([torch.cat(list(self._routing[l])) for l in layers]).cpu()
                record["routing"] = f"{step}.routing.i32"
                self._top_k = int(chosen.shape[2])
                chosen.numpy().astype("<i4", copy=False).tofile(os.path.join(self.out_dir, record["routing"]))
            eng.check_device_errors()
        for rid in obj.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                eng.release_slot(self.slots.pop(rid))
        self.index.append(record)

    def close(self) -> None:
        eng = self.engine
        routed = sorted(self._routing) if self._routing else []
        meta = {"vocab_size": eng.spec.vocab_size, "dtype": str(eng.dtype).replace("torch.", ""),
                "routed_layers": routed, "top_k": self._top_k, "steps": self.index}
        tmp = os.path.join(self.out_dir, "index.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f)
        os.replace(tmp, os.path.join(self.out_dir, "index.json"))
        if self._routing is not None:
            eng.capture_routing(False)
