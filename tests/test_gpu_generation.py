"""Generation through the Python entry point and the command line, and sampling on the device."""
import os
import subprocess
import sys

import pytest
import torch

import plain_llama4 as P
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def dirs():
    return {n: tiny.make_model_dir(n) for n in "AB"}


@pytest.mark.parametrize("name,lengths,steps,dtype", [
    ("A", (5, 17, 40), 24, "float32"), ("B", (1, 9, 33, 70), 16, "float32"),
    ("A", (5, 17, 40), 24, "bfloat16"), ("B", (1, 9, 33, 70), 16, "bfloat16"), ("C", (5, 70, 150), 12, "bfloat16")])
def test_greedy_generation_matches_plain(dirs, name, lengths, steps, dtype):
    """Every generated token is the plain implementation's best token for the sequence so far, or so close to
    it that the precision's rounding decides (twice the logit tolerance: both logits may be off by it)."""
    from cpi_b200.api import Model
    from helpers import tolerances
    if name not in dirs:
        dirs[name] = tiny.make_model_dir(name)
    d = dirs[name]
    c, W = P.read_config(d), P.read_weights(d)
    prompts = [tiny.random_tokens(n, c["vocab_size"], 7 * n + 1) for n in lengths]
    m = Model.load(d, dtype=dtype, max_batch=len(prompts), max_context=256)
    got = m.generate(prompts, max_new=steps, temperature=0.0, stop_ids=[])
    tol = tolerances(dtype)[0] * (1 if dtype == "float32" else 2)
    parted = 0
    for p, g in zip(prompts, got):
        seq = list(p)
        for i, tok in enumerate(g.tokens):
            lg = P.forward(c, W, seq)[-1]
            best = int(torch.argmax(lg))
            if tok != best:        # only a near-tie of the two logits may part the two
                parted += 1
                assert float(lg[best] - lg[tok]) <= tol * float(lg.abs().max()), (i, tok, best)
            seq.append(tok)
        assert g.finish_reason == "max_new" and len(g.tokens) == steps
    print(f"greedy generation {name} {dtype}: {parted} of {steps * len(prompts)} tokens were near-ties taken "
          f"the other way")
    assert m.stats().generated_tokens == steps * len(prompts)
    assert not m.engine.cache.live_slots()


def test_stop_tokens_end_sequences_early_and_more_requests_than_slots(dirs):
    from cpi_b200.api import Model
    d = dirs["A"]
    c, W = P.read_config(d), P.read_weights(d)
    prompts = [tiny.random_tokens(n, 512, 90 + n) for n in (3, 8, 21, 13, 6)]
    m = Model.load(d, dtype="float32", max_batch=2, max_context=64)
    free = m.generate(prompts, max_new=8, temperature=0.0, stop_ids=[])
    stop = free[0].tokens[2]
    got = m.generate(prompts, max_new=8, temperature=0.0, stop_ids=[stop])
    assert m.stats().batches == 3
    for f, g in zip(free, got):
        if stop in f.tokens:
            cut = f.tokens.index(stop) + 1
            assert g.tokens == f.tokens[:cut] and g.finish_reason == "stop_token"
        else:
            assert g.tokens == f.tokens and g.finish_reason == "max_new"
    assert got[0].tokens == free[0].tokens[:3]
    m.engine.cache.check_consistency()


def test_temperature_sampling_is_reproducible_and_follows_the_distribution(dirs):
    from cpi_b200.sampling import SamplingParams
    from cpi_b200.sampling.sampler import Sampler
    dev = torch.device("cuda:0")
    V = 11
    s = Sampler(dev, V)
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -2.0, 0.0, 0.3, -0.5, 1.2])
    T = 0.7
    N = 4000
    sp = SamplingParams(temperature=T, top_k=V, top_p=1.0, seed=11)
    rows = logits.repeat(N, 1).to(dev)
    a = s.sample(rows.clone(), [sp] * N, [[]] * N, [(0, i) for i in range(N)])
    b = s.sample(rows.clone(), [sp] * N, [[]] * N, [(0, i) for i in range(N)])
    assert a == b
    c = s.sample(rows.clone(), [SamplingParams(temperature=T, top_k=V, top_p=1.0, seed=12)] * N, [[]] * N,
                 [(0, i) for i in range(N)])
    assert a != c
    p = torch.softmax(logits / T, 0)
    freq = torch.bincount(torch.tensor(a), minlength=V).float() / N
    assert float((freq - p).abs().max()) < 4.0 * float((p * (1 - p) / N).sqrt().max())
    # top-k 3 keeps ids 0, 5, 10; top-p cuts further
    k3 = s.sample(rows.clone(), [SamplingParams(temperature=T, top_k=3, top_p=1.0, seed=1)] * N, [[]] * N,
                  [(0, i) for i in range(N)])
    assert set(k3) == {0, 5, 10}
    p3 = p[[0, 5, 10]] / p[[0, 5, 10]].sum()
    f3 = torch.tensor([k3.count(0), k3.count(5), k3.count(10)]).float() / N
    assert float((f3 - p3).abs().max()) < 0.04
    cum = float(p[0] + p[5])
    pp = s.sample(rows.clone(), [SamplingParams(temperature=T, top_k=V, top_p=cum - 1e-3, seed=1)] * N, [[]] * N,
                  [(0, i) for i in range(N)])
    assert set(pp) == {0, 5}
    # greedy takes the first maximum; the penalty and the n-gram ban act before it
    tie = torch.tensor([[0.0, 3.0, 3.0, 1.0]], device=dev)
    g0 = SamplingParams(temperature=0.0)
    assert Sampler(dev, 4).sample(tie.clone(), [g0], [[]], [(0, 0)]) == [1]
    pen = SamplingParams(temperature=0.0, repetition_penalty=2.0)
    assert Sampler(dev, 4).sample(tie.clone(), [pen], [[1, 1, 0]], [(0, 0)]) == [2]
    ban = SamplingParams(temperature=0.0, no_repeat_ngram_size=2)
    assert Sampler(dev, 4).sample(tie.clone(), [ban], [[3, 1, 0, 3]], [(0, 0)]) == [2]
    bad = torch.tensor([[float("nan"), float("inf"), 100.0, -5.0]], device=dev)
    assert Sampler(dev, 4).sample(bad, [SamplingParams(temperature=0.0, repetition_penalty=1.5)], [[3]], [(0, 0)]) == [2]


def test_command_line_prints_the_reference_lines(dirs):
    d = dirs["A"]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), d, "--tokens", "5,6,7",
                        "--max-new", "4", "--temp", "0", "--dtype", "float32", "--eos-token", "-1", "--benchmark",
                        "--inspect-next-topk", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    c, W = P.read_config(d), P.read_weights(d)
    want = P.greedy_generate(c, W, [5, 6, 7], 4)
    lines = r.stdout.splitlines()
    out = [l for l in lines if l.startswith("Output tokens:")][0]
    assert out.split(":")[1].split() == [str(t) for t in [5, 6, 7] + want]
    assert any(l.startswith("[perf] generated_tokens=4 ") for l in lines)
    assert any(l.startswith("[bench] prefill_tokens=2 ") and "decode_tok_per_s=" in l for l in lines)
    top = [l for l in lines if l.startswith("  id=")]
    assert len(top) == 3 and top[0].startswith(f"  id={want[0]} logit=")
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), d + "_missing", "--temp", "0"],
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode == 2 and "fatal" in bad.stderr


def test_command_line_overrides_presets_phases_and_logits(dirs, tmp_path):
    """--preset and --rope-theta reach the configuration (the plain implementation is given the same keys),
    --dump-logits writes the rows after the prompts, repeated runs print the -avg lines and --benchmark-phases
    one figure for each of the reference's phase names."""
    import numpy as np
    from cpi_b200.config.llama4 import PRESETS
    d = dirs["A"]
    f = str(tmp_path / "logits.f32")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), d, "--tokens", "9,8,7,6,5",
                        "--max-new", "5", "--temp", "0", "--dtype", "float32", "--eos-token", "-1",
                        "--preset", "reference_compat", "--rope-theta", "10000", "--rope-pairing", "interleaved",
                        "--benchmark-reps", "2", "--benchmark-phases", "--dump-logits", f],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    c, W = P.read_config(d), P.read_weights(d)
    c.update(PRESETS["reference_compat"], rope_theta=10000.0, rope_pairing="interleaved")
    want = P.greedy_generate(c, W, [9, 8, 7, 6, 5], 5)
    lines = r.stdout.splitlines()
    out = [l for l in lines if l.startswith("Output tokens:")][0]
    assert out.split(":")[1].split() == [str(t) for t in [9, 8, 7, 6, 5] + want]
    plain_logits = P.forward(c, W, [9, 8, 7, 6, 5])[-1]
    got = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(1, -1))[0]
    assert float((got - plain_logits).abs().max()) <= 2e-4 * float(plain_logits.abs().max())
    # the overrides matter: without them the same prompt gives other logits
    assert float((P.forward(P.read_config(d), W, [9, 8, 7, 6, 5])[-1] - plain_logits).abs().max()) > 1e-2
    assert any(l.startswith("[perf-avg] generated_tokens=5 ") for l in lines)
    assert any(l.startswith("[bench-avg] reps=2 prefill_tokens=4 ") and "total_tok_per_s=" in l for l in lines)
    phase = [l for l in lines if l.startswith("[bench-phase-avg] ")]
    assert len(phase) == 1
    fields = dict(x.split("=") for x in phase[0].split()[1:])
    assert list(fields) == [n + "_ms" for n in ("rmsnorm", "qkv", "kv_store", "attention", "wo", "mlp", "moe_router",
                                                "moe_expert", "moe_merge", "lm_head")]
    for name in ("rmsnorm_ms", "qkv_ms", "kv_store_ms", "attention_ms", "wo_ms", "moe_router_ms", "moe_expert_ms",
                 "lm_head_ms"):
        assert float(fields[name]) > 0.0, name


def test_run_llama4_prompt_script(dirs):
    d = dirs["B"]
    c, W = P.read_config(d), P.read_weights(d)
    want = P.greedy_generate(c, W, [7, 7, 2], 8)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_llama4_prompt"), d, "7,7,2", "--max-new", "8",
                        "--dtype", "float32", "--stop-ids", str(want[4])], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    first = want.index(want[4])
    assert [l for l in lines if l.startswith("Output tokens:")][0].split(":")[1].split() == \
        [str(t) for t in [7, 7, 2] + want[:first + 1]]                  # the stop token ends generation and is kept
    assert [l for l in lines if l.startswith("Answer tokens:")][0].split(":")[1].split() == \
        [str(t) for t in want[:first]]
    text = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_llama4_prompt"), d, "hello there"],
                          capture_output=True, text=True, timeout=300)
    assert text.returncode == 1 and "token ids" in text.stderr


def test_interactive_mode_speaks_json_lines(dirs):
    import json
    d = dirs["B"]
    c, W = P.read_config(d), P.read_weights(d)
    want = P.greedy_generate(c, W, [3, 1, 4, 1, 5], 6)
    requests = [{"id": "r1", "tokens": [3, 1, 4, 1, 5], "max_new": 6, "temp": 0, "stop_ids": []},
                {"id": "r2", "tokens": [3, 1, 4, 1, 5], "max_new": 6, "temp": 0, "stop_ids": [want[2]]},
                {"id": "r3", "max_new": 2},
                {"id": "bye", "shutdown": True},
                {"id": "never", "tokens": [1]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), d, "--interactive", "--dtype",
                        "float32", "--max-context", "64"], input="".join(json.dumps(q) + "\n" for q in requests),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    ev = [json.loads(l) for l in r.stdout.splitlines()]
    by = lambda rid: [e for e in ev if e.get("id") == rid]
    assert [e["type"] for e in by("r1")] == ["start"] + ["delta", "metrics"] * 6 + ["done"]
    assert [e["tokens"][0] for e in by("r1") if e["type"] == "delta"] == want
    assert [e["metrics"]["token_index"] for e in by("r1") if e["type"] == "metrics"] == [1, 2, 3, 4, 5, 6]
    done = by("r1")[-1]
    assert done["tokens"] == want and done["generated_tokens"] == 6 and done["elapsed_ms"] >= 0
    assert by("r2")[-1]["tokens"] == want[:want.index(want[2])]          # the stop token is not part of the answer
    assert [e["type"] for e in by("r3")] == ["error"] and "tokens" in by("r3")[0]["error"]
    assert [e["type"] for e in by("bye")] == ["done"] and not by("never")


def test_phase_timer_on_the_engine(dirs):
    """Phases are timed for prefill and decode steps; switching the timer off brings the graphs back, and
    the logits are the same with and without it."""
    from cpi_b200.engine import Engine, StepEntry
    e = Engine.from_model_dir(tiny.make_model_dir("C"), dtype="bfloat16", max_tokens=256)
    t = tiny.random_tokens(30, 777, 5)

    def run():
        s = e.acquire_slot()
        rows = [e.step([StepEntry(s, t[:20], [19])]).clone()]
        for x in t[20:]:
            rows.append(e.step([StepEntry(s, [x], [0])]).clone())
        e.release_slot(s)
        return torch.cat(rows)

    plain_run = run()
    assert e._graphs
    timer = e.profile_phases(True)
    timed = run()
    ms = timer.collect()
    e.profile_phases(False)
    assert torch.equal(plain_run, timed)
    assert set(ms) == {"prefill", "decode"}
    for kind in ms:
        assert {"embedding", "rmsnorm", "qkv", "kv_store", "attention", "wo", "mlp", "moe_router", "moe_expert",
                "moe_merge", "lm_head"} == set(ms[kind]), ms[kind].keys()
        assert all(v > 0 for v in ms[kind].values())
    from cpi_b200 import phases
    assert phases.active() is None
    assert torch.equal(run(), plain_run)


def test_trace_run_program(dirs, tmp_path):
    """bin/trace_run on a two-request trace, in float32, against the plain implementation."""
    import json
    import numpy as np
    d = dirs["B"]
    c, W = P.read_config(d), P.read_weights(d)
    a, b = tiny.random_tokens(40, 1000, 1), tiny.random_tokens(12, 1000, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]},
                                     {"id": "b", "tokens": b[:11], "want": [10]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[37]], "want": [0]},
                                     {"id": "b", "tokens": [b[11]], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[38]], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[39]], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "3.f32", "index.json"]
    la, lb = P.forward(c, W, a).numpy(), P.forward(c, W, b).numpy()
    s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, 1000)
    s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, 1000)
    s3 = np.fromfile(out / "3.f32", dtype="<f4").reshape(1, 1000)
    scale = np.abs(la).max()
    for got, want in ((s0[0], la[0]), (s0[1], la[36]), (s0[2], lb[10]), (s1[0], la[37]), (s3[0], la[39])):
        assert np.abs(got - want).max() <= 2e-5 * scale
