"""Test helpers: drive the engine through a schedule of steps and compare with the plain implementation."""
from __future__ import annotations

import torch

import plain_llama4 as P


def tolerances(dtype: str):
    """(logit tolerance relative to max |logit|, router near-tie tolerance relative to max |router logit|)."""
    if dtype == "float32":
        return 2e-5, 1e-4
    return 2e-2, 4e-2


class Replay:
    """Runs requests through an engine and records logits and expert choices per (request, position)."""

    def __init__(self, engine):
        self.e = engine
        self.logits = {}      # rid -> {pos: tensor [V] (cpu)}
        self.routing = {}     # rid -> {layer: {pos: [k]}}
        self.slots = {}
        self.cap = engine.capture_routing(True)

    def step(self, items):
        """items: list of (rid, tokens, want) -- want = places among these tokens."""
        from cpi_b200.engine import StepEntry
        entries, layout = [], []
        for rid, toks, want in items:
            if rid not in self.slots:
                self.slots[rid] = self.e.acquire_slot()
            start = self.e.length(self.slots[rid])
            entries.append(StepEntry(self.slots[rid], toks, want))
            layout.append((rid, start, len(toks), list(want)))
        for lst in self.cap.values():
            lst.clear()
        out = self.e.step(entries).float().cpu()
        self.e.check_device_errors()
        r = 0
        for rid, start, n, want in layout:
            for w in want:
                self.logits.setdefault(rid, {})[start + w] = out[r]
                r += 1
        for layer, lst in self.cap.items():
            # a step larger than the engine's max_step_tokens runs as pieces, each of which records its own
            # tokens' choices; the pieces follow the packed order, so joined they are the step's
            idx = torch.cat([x.cpu() for x in lst])
            assert idx.shape[0] == sum(n for _, _, n, _ in layout)
            t = 0
            for rid, start, n, _ in layout:
                for i in range(n):
                    self.routing.setdefault(rid, {}).setdefault(layer, {})[start + i] = idx[t + i].tolist()
                t += n

    def end(self, rid):
        self.e.release_slot(self.slots.pop(rid))


def compare_with_plain(model_dir, requests, replay, dtype, positions=None):
    """requests: {rid: tokens}.  Checks every recorded logit row against the plain implementation run
    with the engine's expert choices, and that every choice that differs from the plain one was a
    near-tie of the plain router logits.  Returns the largest relative error seen."""
    c, W = P.read_config(model_dir), P.read_weights(model_dir)
    rtol, tie_tol = tolerances(dtype)
    K = c["num_experts_per_tok"]
    worst = 0.0
    for rid, toks in requests.items():
        n = len(toks)
        forced = {}
        for layer, by_pos in replay.routing.get(rid, {}).items():
            assert sorted(by_pos) == list(range(n)), f"routing of {rid} layer {layer} is incomplete"
            forced[layer] = torch.tensor([by_pos[p] for p in range(n)])
        logits, routing = P.forward(c, W, toks, return_router=True, forced_routing=forced or None)
        for layer, r in enumerate(routing):
            if r is None:
                continue
            rl, own = r                       # own = the plain router's choice before forcing
            top = torch.sort(rl, dim=-1, descending=True).values
            scale = float(rl.abs().max())
            for p in range(n):
                chosen = forced[layer][p].tolist()
                kth = float(top[p, K - 1])
                for e in chosen:
                    gap = kth - float(rl[p, e])
                    assert gap <= tie_tol * scale, (
                        f"request {rid} layer {layer} position {p}: engine chose expert {e} whose router "
                        f"logit is {gap:.3e} below the k-th best (scale {scale:.3e})")
        scale = float(logits.abs().max())
        got = replay.logits.get(rid, {})
        check = sorted(got) if positions is None else positions[rid]
        assert check, f"no logits recorded for {rid}"
        for p in check:
            err = float((got[p] - logits[p]).abs().max()) / scale
            worst = max(worst, err)
            assert err <= rtol, (f"request {rid} position {p}: logits differ from the plain implementation "
                                 f"by {err:.3e} of max |logit| (tolerance {rtol:.1e}, dtype {dtype})")
    return worst


# ---- the three schedules of the replay tests -----------------------------------------------------------
def run_whole(rp, reqs):
    """Each request alone, its whole token list in one step, logits at every position."""
    for rid, toks in reqs.items():
        rp.step([(rid, toks, list(range(len(toks))))])
        rp.end(rid)


def run_tail(rp, reqs, tail=32):
    """Each request alone: all but the last `tail` tokens in one step, the rest one by one.  Returns the
    positions whose logits were recorded."""
    positions = {}
    for rid, toks in reqs.items():
        n = len(toks)
        head = n - tail
        assert head >= 1
        rp.step([(rid, toks[:head], [head - 1])])
        for i in range(head, n):
            rp.step([(rid, [toks[i]], [0])])
        rp.end(rid)
        positions[rid] = list(range(head - 1, n))
    return positions


def run_batched(rp, batches):
    """batches: a list of {rid: (tokens, prompt_len)}.  In a batch all requests start together with their
    prompts, then bring one token each per step; a request whose tokens are used up ends and leaves the
    batch.  Batch follows batch on the same engine, so slots and pages are used again.  Returns the
    positions whose logits were recorded."""
    e = rp.e
    positions = {}
    for reqs in batches:
        rp.step([(rid, t[:p], [p - 1]) for rid, (t, p) in reqs.items()])
        live = dict(reqs)
        step = 0
        while live:
            for rid in [r for r, (t, p) in live.items() if p + step >= len(t)]:
                rp.end(rid)
                del live[rid]
            if not live:
                break
            rp.step([(rid, [t[p + step]], [0]) for rid, (t, p) in live.items()])
            step += 1
        e.cache.check_consistency()
        assert e.cache.free_slots == e.cache.max_slots
        for rid, (t, p) in reqs.items():
            positions[rid] = list(range(p - 1, len(t)))
    return positions


class TraceOutput:
    """What `bin/trace_run` wrote into a folder, in the shape `compare_with_plain` reads: logits per (request,
    position) and, when the tool dumped them, expert choices per (request, layer, position)."""

    def __init__(self, out_dir):
        import json
        import os
        import numpy as np
        with open(os.path.join(out_dir, "index.json")) as f:
            idx = json.load(f)
        V, layers, k = idx["vocab_size"], idx["routed_layers"], idx["top_k"]
        self.logits, self.routing, self.steps = {}, {}, idx["steps"]
        for st in idx["steps"]:
            rows = sum(len(e["want"]) for e in st["entries"])
            assert (st["file"] is not None) == (rows > 0)
            if rows:
                arr = np.fromfile(os.path.join(out_dir, st["file"]), dtype="<f4")
                assert arr.size == rows * V, f"step {st['step']}: {arr.size} floats for {rows} rows"
                lg = torch.from_numpy(arr.reshape(rows, V).copy())
                r = 0
                for e in st["entries"]:
                    for w in e["want"]:
                        self.logits.setdefault(e["id"], {})[e["start"] + w] = lg[r]
                        r += 1
            if st["routing"]:
                T = sum(e["tokens"] for e in st["entries"])
                ch = np.fromfile(os.path.join(out_dir, st["routing"]), dtype="<i4").reshape(len(layers), T, k)
                t = 0
                for e in st["entries"]:
                    for i in range(e["tokens"]):
                        for li, layer in enumerate(layers):
                            self.routing.setdefault(e["id"], {}).setdefault(layer, {})[e["start"] + i] = \
                                ch[li, t + i].tolist()
                    t += e["tokens"]
