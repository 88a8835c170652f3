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


@pytest.mark.parametrize("name,lengths,steps", [("A", (5, 17, 40), 24), ("B", (1, 9, 33, 70), 16)])
def test_greedy_generation_matches_plain_in_float32(dirs, name, lengths, steps):
    from cpi_b200.api import Model
    d = dirs[name]
    c, W = P.read_config(d), P.read_weights(d)
    prompts = [tiny.random_tokens(n, c["vocab_size"], 7 * n + 1) for n in lengths]
    m = Model.load(d, dtype="float32", max_batch=len(prompts), max_context=128)
    got = m.generate(prompts, max_new=steps, temperature=0.0, stop_ids=[])
    for p, g in zip(prompts, got):
        seq = list(p)
        for i, tok in enumerate(g.tokens):
            lg = P.forward(c, W, seq)[-1]
            best = int(torch.argmax(lg))
            if tok != best:        # only a near-tie of the two best logits may part the two
                assert float(lg[best] - lg[tok]) <= 2e-5 * float(lg.abs().max()), (i, tok, best)
            seq.append(tok)
        assert g.finish_reason == "max_new" and len(g.tokens) == steps
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
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "3.f32"]
    la, lb = P.forward(c, W, a).numpy(), P.forward(c, W, b).numpy()
    s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, 1000)
    s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, 1000)
    s3 = np.fromfile(out / "3.f32", dtype="<f4").reshape(1, 1000)
    scale = np.abs(la).max()
    for got, want in ((s0[0], la[0]), (s0[1], la[36]), (s0[2], lb[10]), (s1[0], la[37]), (s3[0], la[39])):
        assert np.abs(got - want).max() <= 2e-5 * scale
