"""The generation loop's decisions, on a fake engine: order of stop checks, batches, slot reuse."""
from dataclasses import dataclass

import pytest

from cpi_b200.engine.generate import GenerationRequest, Generator, plan_batches
from cpi_b200.sampling import SamplingParams
from cpi_b200.sampling.sampler import banned_by_ngram, uniform_for


@dataclass
class Entry:
    slot: int
    tokens: list
    want: list


class FakeCache:
    def __init__(self, n_pages, page_size, max_seq_len):
        self.n_pages, self.page_size, self.max_seq_len = n_pages, page_size, max_seq_len


class FakeEngine:
    """next token = (last token + 1) % vocab; records every step; checks slot discipline."""

    def __init__(self, slots=4, n_pages=64, page_size=16, max_seq_len=256, vocab=50):
        self.cache = FakeCache(n_pages, page_size, max_seq_len)
        self.free = list(range(slots))
        self.live = {}
        self.steps = []
        self.vocab = vocab
        self.acquired = []

    def acquire_slot(self):
        s = self.free.pop(0)
        self.live[s] = []
        self.acquired.append(s)
        return s

    def release_slot(self, s):
        assert s in self.live, "released twice"
        del self.live[s]
        self.free.append(s)

    def step(self, entries):
        self.steps.append([(e.slot, list(e.tokens)) for e in entries])
        out = []
        for e in entries:
            assert e.slot in self.live
            if self.live[e.slot]:
                assert len(e.tokens) == 1, "a started sequence goes on by one token"
            self.live[e.slot] += list(e.tokens)
            assert len(self.live[e.slot]) <= self.cache.max_seq_len
            for _ in e.want:
                out.append((self.live[e.slot][-1] + 1) % self.vocab)
        return out


class FakeSampler:
    def sample(self, logits, params, histories, counters):
        self.last = (params, histories, counters)
        return list(logits)


def gen(engine, **kw):
    return Generator(engine, FakeSampler(), step_entry=Entry, **kw)


class AheadEngine(FakeEngine):
    """The fake engine with the call that takes its tokens from a tensor, as the loop that runs one step
    ahead of the host uses it."""

    def step_decode(self, slots, tokens):
        toks = tokens.tolist()
        assert len(toks) == len(slots)
        return self.step([Entry(s, [t], [0]) for s, t in zip(slots, toks)])


class AheadSampler(FakeSampler):
    def sample_device(self, logits, params, histories, counters):
        import torch
        self.last = (params, histories, counters)
        return torch.tensor(list(logits), dtype=torch.int32)


def gen_ahead(engine, **kw):
    return Generator(engine, AheadSampler(), step_entry=Entry, **kw)


def test_stop_token_is_kept_and_ends_the_sequence():
    e = FakeEngine()
    g = gen(e, max_batch=4, default_stop_ids=[13])
    r = g.generate([GenerationRequest([10], 20), GenerationRequest([1, 2, 3], 4)])
    assert r[0].tokens == [11, 12, 13] and r[0].finish_reason == "stop_token"
    assert r[1].tokens == [4, 5, 6, 7] and r[1].finish_reason == "max_new" and r[1].prompt_tokens == 3
    assert not e.live and sorted(e.free) == [0, 1, 2, 3]
    # prompts run in one step; afterwards one token each; the finished request leaves the batch
    assert e.steps[0] == [(0, [10]), (1, [1, 2, 3])]
    assert e.steps[1] == [(0, [11]), (1, [4])] and e.steps[2] == [(0, [12]), (1, [5])]
    assert e.steps[3] == [(1, [6])] and len(e.steps) == 4
    assert g.stats.generated_tokens == 7 and g.stats.prompt_tokens == 4 and g.stats.decode_steps == 3


def test_request_stop_ids_override_the_models():
    e = FakeEngine()
    g = gen(e, max_batch=2, default_stop_ids=[5])
    r = g.generate([GenerationRequest([3], 6, stop_ids=[]), GenerationRequest([3], 6, stop_ids=[7])])
    assert r[0].tokens == [4, 5, 6, 7, 8, 9] and r[0].finish_reason == "max_new"
    assert r[1].tokens == [4, 5, 6, 7] and r[1].finish_reason == "stop_token"


def test_callback_stops_after_the_token_is_appended_and_stop_token_wins():
    e = FakeEngine()
    g = gen(e, max_batch=2, default_stop_ids=[6])
    seen = []

    def cb(i, tok):
        seen.append((i, tok))
        return tok != 5

    r = g.generate([GenerationRequest([3], 9), GenerationRequest([5], 9)], cb)
    assert r[0].tokens == [4, 5] and r[0].finish_reason == "callback"
    assert r[1].tokens == [6] and r[1].finish_reason == "stop_token"
    assert (1, 6) in seen and (0, 5) in seen      # the callback sees the end token too; the reason stays the token


def test_max_context_is_the_callers_figure_not_the_cache_rounded_up():
    e = FakeEngine(max_seq_len=128, page_size=64, n_pages=8)       # a cache of whole pages: 128 positions
    g = gen(e, max_batch=1, max_context=100)
    r = g.generate([GenerationRequest(list(range(40)), 500)])
    assert r[0].finish_reason == "capacity" and len(r[0].tokens) == 61      # 40 + 61 - 1 == 100 positions run
    assert len(e.steps) == 61
    with pytest.raises(ValueError, match="longest"):
        g.generate([GenerationRequest(list(range(101)), 2)])
    g.generate([GenerationRequest(list(range(100)), 2)])


def test_capacity_stop():
    e = FakeEngine(max_seq_len=8, page_size=4, n_pages=8)
    g = gen(e, max_batch=1)
    r = g.generate([GenerationRequest([0, 1, 2, 3, 4], 50)])
    assert r[0].finish_reason == "capacity" and r[0].tokens == [5, 6, 7, 8]
    with pytest.raises(ValueError, match="longest"):
        g.generate([GenerationRequest(list(range(9)), 2)])


def test_batches_follow_each_other_in_freed_slots():
    e = FakeEngine(slots=2)
    g = gen(e, max_batch=2)
    r = g.generate([GenerationRequest([i], 2 + i) for i in range(5)])
    assert [x.tokens for x in r] == [[(i + 1 + j) % 50 for j in range(2 + i)] for i in range(5)]
    assert g.stats.batches == 3 and e.acquired == [0, 1, 0, 1, 1] or e.acquired[:2] == [0, 1]
    assert len(e.acquired) == 5 and set(e.acquired) == {0, 1} and not e.live


def test_plan_batches_respects_cache_tokens():
    reqs = [GenerationRequest([0] * p, m) for p, m in [(10, 7), (33, 1), (60, 5), (5, 5)]]
    # needs, rounded to pages of 16: 16, 48, 64, 16
    assert plan_batches(reqs, max_batch=8, token_capacity=128, page_size=16, max_seq_len=999) == [[0, 1, 2], [3]]
    assert plan_batches(reqs, max_batch=2, token_capacity=1 << 20, page_size=16, max_seq_len=999) == [[0, 1], [2, 3]]
    with pytest.raises(ValueError, match="cache holds"):
        plan_batches(reqs, max_batch=2, token_capacity=48, page_size=16, max_seq_len=999)


def test_empty_prompt_uses_bos_or_fails():
    e = FakeEngine()
    with pytest.raises(ValueError, match="empty prompt"):
        gen(e, max_batch=1).generate([GenerationRequest([], 2)])
    r = gen(e, max_batch=1, bos_token_id=9).generate([GenerationRequest([], 2)])
    assert r[0].tokens == [10, 11] and r[0].prompt_tokens == 1


def test_slots_are_returned_when_a_step_fails():
    e = FakeEngine()

    def boom(entries):
        raise RuntimeError("step failed")

    g = gen(e, max_batch=2)
    e.step = boom
    with pytest.raises(RuntimeError):
        g.generate([GenerationRequest([1], 2), GenerationRequest([2], 2)])
    assert not e.live and len(e.free) == 4


def test_sampler_receives_histories_and_counters():
    e = FakeEngine()
    g = gen(e, max_batch=2)
    sp = SamplingParams(temperature=0.7, seed=3, repetition_penalty=1.2)
    g.generate([GenerationRequest([1, 2], 3, sp), GenerationRequest([7], 2, sp)])
    params, hist, counters = g.sampler.last
    assert hist == [[1, 2, 3, 4]] and counters == [(0, 2)] and params == [sp]
    # histories are only built for the options that read them (they grow with the context)
    sp = SamplingParams(temperature=0.7, seed=3)
    g.generate([GenerationRequest([1, 2], 3, sp)])
    params, hist, counters = g.sampler.last
    assert hist == [None] and counters == [(0, 2)] and params == [sp]


def test_ngram_bans_and_uniforms():
    assert banned_by_ngram([1, 2, 3, 1, 2], 3) == [3]
    assert banned_by_ngram([1, 2, 1, 3, 1], 2) == [2, 3]
    assert banned_by_ngram([1, 2], 4) == [] and banned_by_ngram([1, 2, 3], 1) == []
    u = uniform_for(5, 1, 2)
    assert 0.0 <= u < 1.0 and u == uniform_for(5, 1, 2)
    assert len({uniform_for(5, 1, s) for s in range(20)} | {uniform_for(6, 1, 2)}) == 21


def test_sampling_params_validation():
    SamplingParams(temperature=0.0, top_k=100000).validate()
    with pytest.raises(ValueError, match="top_k"):
        SamplingParams(temperature=1.0, top_k=1000).validate()
    with pytest.raises(ValueError):
        SamplingParams(repetition_penalty=0.0).validate()
    assert SamplingParams(temperature=0.0).is_plain_greedy
    assert not SamplingParams(temperature=0.0, repetition_penalty=1.2).is_plain_greedy


SCENARIOS = [
    dict(reqs=[([10], 20), ([1, 2, 3], 4)], stop=[13], eng={}),
    dict(reqs=[([3], 6), ([3], 1), ([40], 30), ([7, 8], 5)], stop=[45, 9], eng={}),
    dict(reqs=[([0, 1, 2, 3, 4], 50)], stop=[], eng=dict(max_seq_len=8, page_size=4, n_pages=8)),
    dict(reqs=[([i], 2 + i) for i in range(5)], stop=[4], eng=dict(slots=2), max_batch=2),
    dict(reqs=[([5], 1), ([6], 1)], stop=[], eng={}),
]


@pytest.mark.parametrize("sc", SCENARIOS)
def test_one_step_ahead_loop_decides_like_the_plain_loop(sc):
    """Same tokens, reasons and slot discipline whether the host reads a step's tokens before the next
    step is launched or after; the loop that runs ahead may spend one step more on a request that ended
    on a stop token, never more."""
    reqs = [GenerationRequest(list(p), m) for p, m in sc["reqs"]]
    e0, e1 = FakeEngine(**sc["eng"]), AheadEngine(**sc["eng"])
    mb = sc.get("max_batch", 4)
    g0, g1 = gen(e0, max_batch=mb, default_stop_ids=sc["stop"]), gen_ahead(e1, max_batch=mb, default_stop_ids=sc["stop"])
    r0, r1 = g0.generate(reqs), g1.generate(reqs)
    assert [(r.tokens, r.finish_reason, r.prompt_tokens) for r in r0] == [(r.tokens, r.finish_reason, r.prompt_tokens) for r in r1]
    assert not e1.live and sorted(e1.free) == sorted(e0.free)
    assert g1.stats.generated_tokens == g0.stats.generated_tokens and g1.stats.batches == g0.stats.batches
    stopped = sum(r.finish_reason == "stop_token" for r in r0)
    assert g0.stats.decode_steps <= g1.stats.decode_steps <= g0.stats.decode_steps + stopped
    # every request's tokens went through the engine in order, one at a time after the prompt
    fed0 = sorted(tuple(t) for st in e0.steps for _, t in st)
    fed1 = sorted(tuple(t) for st in e1.steps for _, t in st)
    assert len(fed1) - len(fed0) <= stopped and all(x in fed1 for x in fed0)


def test_one_step_ahead_loop_is_left_for_callbacks_and_history_options():
    e = AheadEngine()
    g = gen_ahead(e, max_batch=2)
    calls = []
    g.sampler.sample = lambda *a: (calls.append("host"), FakeSampler.sample(g.sampler, *a))[1]
    g.generate([GenerationRequest([1], 3)], lambda i, t: True)
    g.generate([GenerationRequest([1], 3, SamplingParams(temperature=0.5, repetition_penalty=1.3))])
    assert len(calls) == 6
    g.generate([GenerationRequest([1], 3)])
    assert len(calls) == 6                        # plain requests run ahead: sample_device, not sample


def test_command_line_argument_errors_and_interactive_protocol(capsys):
    """What the command line decides without a GPU: flags that need a tokeniser are argument errors (exit 1)
    that name the flag to use, --cpu is a fatal error (exit 2), and the interactive loop's events."""
    import io
    import json
    from cpi_b200.cli import llama_infer as cli
    for argv, word in ((["m", "--prompt", "hi"], "--tokens"), (["m", "--stop-text", "x"], "--stop-ids"),
                       (["m", "--tokenizer", "t.json"], "tokeniser"), (["m", "--rope-theta", "0"], "--rope-theta"),
                       ([], "model folder"), (["m", "--preset", "nope"], "")):
        assert cli.main(argv) == 1
        assert word in capsys.readouterr().err
    assert cli.main(["m", "--cpu"]) == 2 and "no CPU path" in capsys.readouterr().err
    a = cli.build_parser().parse_args(["m", "--preset", "reference_compat", "--router-gate", "sigmoid_output",
                                       "--rope-theta", "1e6", "--benchmark-phases"])
    cli.validate(a)
    assert a.benchmark and cli.config_overrides(a)["router_gate"] == "sigmoid_output"
    assert cli.config_overrides(a)["qk_norm_order"] == "before_rope" and cli.config_overrides(a)["rope_theta"] == 1e6
    assert cli.config_overrides(cli.build_parser().parse_args(["m"])) == {}

    class FakeModel:
        def generate(self, prompts, on_token=None, max_new=0, stop_ids=(), **kw):
            self.kw = dict(kw, max_new=max_new, stop_ids=stop_ids)
            for t in range(10, 10 + max_new):
                if t in stop_ids or not on_token(0, t):
                    break

    m, out = FakeModel(), io.StringIO()
    lines = [json.dumps({"id": "a", "tokens": [1, 2], "max_new": 3, "temp": -1}), "", "not json",
             json.dumps({"id": "b", "tokens": [1], "stop_ids": [11]}), json.dumps({"shutdown": True}),
             json.dumps({"id": "late", "tokens": [1]})]
    defaults = dict(max_new=4, temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.0, no_repeat_ngram_size=0,
                    seed=0, stop_ids=[12])
    assert cli.interactive(m, defaults, io.StringIO("\n".join(lines) + "\n"), out) == 0
    ev = [json.loads(l) for l in out.getvalue().splitlines()]
    assert [e["type"] for e in ev] == ["start", "delta", "metrics", "delta", "metrics", "done", "error", "start",
                                       "delta", "metrics", "done", "done"]
    assert ev[5]["tokens"] == [10, 11] and ev[5]["id"] == "a"       # the default stop id 12 ended it
    assert ev[10]["tokens"] == [10] and "id" not in ev[11]
    assert m.kw["temperature"] == 0.8 and m.kw["max_new"] == 4      # the second request ran on the defaults


def test_command_line_is_one_instance_at_a_time(tmp_path, monkeypatch, capsys):
    """While one process holds the lock file, a second start ends with exit code 3 and the reference's sentence
    (src/main.cpp:51-55); when the first has ended the lock is free again."""
    import fcntl
    import os
    from cpi_b200.cli import llama_infer as cli
    lock = str(tmp_path / "instance.lock")
    monkeypatch.setenv("LLAMA_INFER_LOCK_PATH", lock)
    fd = os.open(lock, os.O_CREAT | os.O_RDWR, 0o644)
    fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
    assert cli.main(["m", "--cpu"]) == 3
    assert "Another llama_infer instance is already running." in capsys.readouterr().err
    fcntl.flock(fd, fcntl.LOCK_UN)
    os.close(fd)
    assert cli.main(["m", "--cpu"]) == 2          # the lock is free: the run gets as far as its own error
    g = cli.SingleInstance()
    assert g.acquire() and not cli.SingleInstance().acquire()
    g.release()
    assert cli.SingleInstance().acquire()


def test_command_line_options_come_from_the_registered_architectures():
    """The command line knows no architecture: presets and model options are what the registry's entries declare,
    and an architecture registered from outside brings its own."""
    from cpi_b200.cli import llama_infer as cli
    from cpi_b200.config import registry
    flags = {o[0] for o in registry.cli_options()}
    assert {"--rope-theta", "--rope-pairing", "--qk-norm-order", "--qk-norm-scope", "--router-gate"} <= flags
    assert {"llama4", "reference_compat"} <= set(registry.cli_presets())
    toy = registry.Architecture("ToyForTests", lambda raw: raw, lambda cfg: None, {"toy_preset": {"toy_width": 3}},
                                (("--toy-depth", "toy_depth", int, "layers of the toy"),))
    registry.register_architecture(toy)
    try:
        a = cli.build_parser().parse_args(["m", "--preset", "toy_preset", "--toy-depth", "5"])
        assert cli.config_overrides(a) == {"toy_width": 3, "toy_depth": 5}
    finally:
        registry._ARCHITECTURES.pop("ToyForTests")


def test_bench_refuses_more_than_one_gpu_and_names_the_reference_arm():
    """What bench.py answers without touching a GPU: one line and exit code 2 for N > 1, and the reference
    arm's `unavailable` line with exit code 0."""
    import json
    import os
    import subprocess
    import sys
    bench = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    many = subprocess.run([sys.executable, bench, "--gpus", "4", "--steps", "2", "--warmup", "1"],
                          capture_output=True, text=True, timeout=120)
    assert many.returncode == 2
    lines = [l for l in many.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["n_gpus"] == 4 and "single-GPU" in lines[0]
    ref = subprocess.run([sys.executable, bench, "--impl", "reference", "--gpus", "1"], capture_output=True, text=True,
                         timeout=120)
    assert ref.returncode == 0
    rec = json.loads(ref.stdout.strip())
    assert rec["impl"] == "reference" and rec["unavailable"]


def test_compare_logits_measures():
    import torch
    from cpi_b200.engine.drift import compare_logits
    ref = torch.tensor([[0.0, 5.0, 4.0, 3.0, -1.0, 2.0], [9.0, 1.0, 2.0, 3.0, 4.0, 5.0]])
    same = compare_logits(ref, ref, 3)
    assert same["top1_match"] == 1.0 and same["overlap_at_k"] == 1.0 and same["mean_abs"] == 0.0 and same["max_abs"] == 0.0
    other = ref.clone()
    other[0, 1], other[0, 2] = 4.0, 5.5            # row 0: another best token, the same three best
    other[1, 5], other[1, 1] = 0.0, 8.0            # row 1: the same best token, one of its three best replaced
    m = compare_logits(ref, other, 3)
    assert m["top1_match"] == 0.5 and abs(m["overlap_at_k"] - (1.0 + 2.0 / 3.0) / 2) < 1e-6
    assert abs(m["max_abs"] - 7.0) < 1e-6 and abs(m["mean_abs"] - (1.0 + 1.5 + 5.0 + 7.0) / 12) < 1e-6
    assert compare_logits(ref[0], ref[0], 100)["overlap_at_k"] == 1.0       # one row, k larger than the vocabulary
    bad = ref.clone()
    bad[0, 0] = float("nan")
    assert compare_logits(ref, bad, 3)["max_abs"] == float("inf")
    with pytest.raises(ValueError):
        compare_logits(ref, ref[:, :4])


def test_step_batch_layout_on_the_host():
    """What a step's index arrays hold for an unequal batch: packed tokens, each token's sequence and
    position, wanted rows as packed indices, and the query tiles of a prefill (256 tokens of one sequence
    at most, the tile with the most keys first)."""
    import torch
    from cpi_b200.engine.batch import BatchStager
    st = BatchStager("cpu")
    toks = [list(range(100, 400)), [7, 8, 9], list(range(1000, 1130))]            # 300, 3 and 130 new tokens
    starts, slots = [0, 50, 200], [4, 0, 9]
    wants = [[0, 299], [], [129]]
    b = st.stage(slots, starts, toks, wants, torch.float32)
    assert (b.n_tokens, b.n_seqs, b.n_want, b.max_new, b.is_decode) == (433, 3, 3, 300, False)
    assert b.tokens.tolist() == toks[0] + toks[1] + toks[2]
    assert b.token_seq.tolist() == [0] * 300 + [1] * 3 + [2] * 130
    assert b.token_pos.tolist() == list(range(300)) + [50, 51, 52] + list(range(200, 330))
    assert b.seq_slot.tolist() == slots and b.seq_start.tolist() == starts and b.seq_new.tolist() == [300, 3, 130]
    assert b.want_rows.tolist() == [0, 299, 303 + 129]
    tiles = list(zip(b.tile_tok0.tolist(), b.tile_rows.tolist()))
    assert sorted(tiles) == [(0, 256), (256, 44), (300, 3), (303, 130)]
    ends = [b.token_pos[t0 + r - 1].item() + 1 for t0, r in tiles]                   # keys each tile may see
    assert ends == sorted(ends, reverse=True) and b.n_q_tiles == 4
    assert b.ctx_bucket == 512 and st.bytes_staged == 4 * (3 * 433 + 3 * 3 + 3 + 2 * 4)
    d = st.stage([4, 9], [300, 330], [[5], [6]], [[0], [0]], torch.float32)
    assert d.is_decode and d.n_q_tiles == 0 and d.token_pos.tolist() == [300, 330] and d.want_rows.tolist() == [0, 1]
    assert b.tokens.tolist() == toks[0] + toks[1] + toks[2]                         # the ring: the step before is intact
    big = st.stage([1], [0], [list(range(5000))], [[4999]], torch.float32)          # the buffers grow
    assert big.n_tokens == 5000 and big.tokens[-1].item() == 4999 and big.ctx_bucket == 8192
    assert BatchStager.words_needed(8, 8, 8) == 56


def test_run_llama4_prompt_helpers():
    """The chat frame is the reference script's (tools/run_llama4_prompt.py:13-23): system and user turns closed
    by <|eot|>, the assistant's header left open; the answer is cut at the first stop id."""
    from cpi_b200.cli.run_llama4_prompt import chat_frame, cut_at_stop
    text = chat_frame("Be brief.", "Hi")
    assert text == ("<|begin_of_text|><|header_start|>system<|header_end|>\n\nBe brief.<|eot|>"
                    "<|header_start|>user<|header_end|>\n\nHi<|eot|><|header_start|>assistant<|header_end|>\n\n")
    assert cut_at_stop([4, 5, 9, 6, 9], {9}) == [4, 5] and cut_at_stop([4, 5], {9}) == [4, 5] and cut_at_stop([], {1}) == []


def test_replay_schedules_feed_every_token_once_and_in_order():
    """The three schedules of the replay tool, on the host: every request's tokens come once and in order, a
    step's requests all start or all go on by one token, a request ends with its last token, and the cache
    figure is the most that is live at a time."""
    from cpi_b200.engine import replay
    reqs = {"a": list(range(100, 170)), "b": [7], "c": list(range(33)), "d": list(range(200, 264)), "e": [1, 2]}
    for name, steps in (("whole", list(replay.schedule_whole(reqs))), ("tail", list(replay.schedule_tail(reqs, 32))),
                        ("batched", list(replay.schedule_batched(reqs, 2, 32)))):
        fed = {rid: [] for rid in reqs}
        ended, live = [], set()
        assert [s["step"] for s in steps] == list(range(len(steps)))
        for s in steps:
            kinds = set()
            for e in s["entries"]:
                assert e["id"] not in ended
                kinds.add("start" if not fed[e["id"]] else "more")
                if fed[e["id"]]:
                    assert len(e["tokens"]) == 1
                assert all(0 <= w < len(e["tokens"]) for w in e["want"])
                fed[e["id"]] += e["tokens"]
                live.add(e["id"])
            assert len(kinds) == 1, f"{name}: a step mixes starting and continuing requests"
            for rid in s["end"]:
                assert fed[rid] == reqs[rid], f"{name}: {rid} ended before its last token"
                ended.append(rid)
                live.discard(rid)
            if name == "batched":
                assert len(live) <= 2
        assert fed == reqs and sorted(ended) == sorted(reqs) and not live
    assert replay.tokens_needed(replay.schedule_whole(reqs)) == 128
    assert replay.tokens_needed(replay.schedule_batched(reqs, 2, 32)) == 128        # a grows to two pages after b has gone
    assert replay.tokens_needed(replay.schedule_batched(reqs, 5, 32)) == 5 * 64     # all five start with a page each
