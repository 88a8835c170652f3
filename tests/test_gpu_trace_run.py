"""The replay tool as a user runs it: `bin/trace_run` in a process of its own, on a trace file, in its three
modes and both precisions, and its files against the plain implementation."""
import os
import subprocess

import pytest

import tiny
from helpers import TraceOutput, compare_with_plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LENGTHS = {"A": (5, 49, 40, 33, 70, 1, 64), "B": (1, 9, 33, 70, 45, 100, 2)}


@pytest.fixture(scope="module")
def dirs():
    return {n: tiny.make_model_dir(n) for n in "AB"}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_file_in_three_modes_against_plain(dirs, tmp_path, name, dtype):
    """Seven requests of unequal lengths (one of a single token, one that fills a page exactly): each whole, each
    with its last 32 tokens one by one, and in groups of three whose cache holds one group only, so that the
    second and third group run in slots and pages that were given back.  The tool's logits and the experts it
    chose are read from its files."""
    from cpi_b200.engine import replay
    d = dirs[name]
    c = tiny.config(name)
    V = c.get("text_config", c)["vocab_size"]
    reqs = {f"r{i}": tiny.random_tokens(n, V, 900 + 17 * i + n) for i, n in enumerate(LENGTHS[name])}
    trace = tmp_path / "trace.txt"
    trace.write_text("# a comment line\n" + "".join(f"{rid}: {' '.join(map(str, t))}\n" for rid, t in reqs.items()))
    assert replay.read_trace(str(trace)) == reqs
    for mode in ("whole", "tail32", "batched"):
        out = tmp_path / mode
        steps = list({"whole": replay.schedule_whole(reqs), "tail32": replay.schedule_tail(reqs),
                      "batched": replay.schedule_batched(reqs, 3)}[mode])
        need = replay.tokens_needed(steps)
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", str(need), "--trace", str(trace), "--mode", mode, "--batch-size", "3",
                            "--dump-routing"], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert r.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
        got = TraceOutput(str(out))
        positions = {rid: sorted(rows) for rid, rows in got.logits.items()}
        if mode == "whole":
            assert positions == {rid: list(range(len(t))) for rid, t in reqs.items()}
        else:
            assert positions == {rid: list(range(max(1, len(t) - 32) - 1, len(t))) for rid, t in reqs.items()}
        worst = compare_with_plain(d, reqs, got, dtype, positions)
        print(f"trace_run {mode} {name} {dtype}: worst relative error {worst:.3e}")
    # a cache that cannot hold the schedule is refused before anything runs
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out",
                        str(tmp_path / "small"), "--max-tokens", "64", "--trace", str(trace), "--mode", "batched"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 2 and "holds up to" in r.stderr
