"""Schedules of the step function that cut the work in further ways, each against the plain implementation:
steps larger than the engine's `max_step_tokens` (they run as pieces), a prompt that goes on top of a cache that
is not empty, the chunk boundary at the benchmark's head size, and the benchmark's layer sizes through the three
replay schedules."""
import shutil

import pytest
import torch

import tiny
from helpers import Replay, compare_with_plain, run_batched, run_tail, run_whole

pytestmark = pytest.mark.gpu

_dirs = {}


def model_dir(name):
    if name not in _dirs:
        _dirs[name] = tiny.make_model_dir(name)
    return _dirs[name]


def vocab(name):
    c = tiny.config(name)
    return c.get("text_config", c)["vocab_size"]


def make_engine(name, dtype, **kw):
    from cpi_b200.engine import Engine
    return Engine.from_model_dir(model_dir(name), dtype=dtype, **kw)


def sparse_want(n):
    return sorted({0, n - 1} | set(range(2, n, 5)))


# (configuration, precision, max_step_tokens): cuts of two tokens, cuts that fall inside a page (64) and inside a
# chunk (A: 32, B: 16, C: 160), and, for C, pieces as long as or longer than a query tile of the prefill kernel
PIECE_CASES = ([(n, "float32", cap) for n in ("A", "B", "R2") for cap in (2, 37)]
               + [(n, "bfloat16", 37) for n in ("A", "B", "R2")]
               + [("C", "bfloat16", cap) for cap in (2, 37, 128, 200)])


@pytest.mark.parametrize("name,dtype,cap", PIECE_CASES)
def test_oversize_steps_run_as_pieces(name, dtype, cap):
    """An unequal batch of prompts longer than `max_step_tokens`, so that the step runs as pieces: sequences that
    share a piece, sequences cut in the middle (inside a page and inside a chunk), a one-token sequence among
    them, a last piece of one token; logits wanted on both sides of every cut.  Then decoding, whose five
    one-token entries are themselves more than two tokens.  In float32 the pieces must also give what a single
    step gives."""
    lengths = (7, 330, 141, 1, 187) if name == "C" else (7, 90, 41, 1, 47)
    extra = 4
    V = vocab(name)
    reqs = {f"s{i}": tiny.random_tokens(n + extra, V, 500 + 13 * i + n) for i, n in enumerate(lengths)}
    need = sum(-(-len(t) // 64) * 64 for t in reqs.values())

    def run(engine):
        rp = Replay(engine)
        items = []
        for i, (rid, t) in enumerate(reqs.items()):
            n = lengths[i]
            items.append((rid, t[:n], list(range(n)) if i % 2 == 0 else sparse_want(n)))
        rp.step(items)
        for j in range(extra):
            rp.step([(rid, [t[lengths[i] + j]], [0]) for i, (rid, t) in enumerate(reqs.items())])
        for rid in reqs:
            rp.end(rid)
        engine.check_device_errors()
        engine.cache.check_consistency()
        assert engine.cache.free_slots == engine.cache.max_slots
        return rp

    e = make_engine(name, dtype, max_tokens=need, max_step_tokens=cap)
    assert sum(lengths) > cap
    steps_before = e.steps_run
    rp = run(e)
    assert e.steps_run - steps_before >= -(-sum(lengths) // cap) + extra * -(-len(lengths) // cap)
    worst = compare_with_plain(model_dir(name), reqs, rp, dtype)
    print(f"pieces of {cap}, {name} {dtype}: worst relative error {worst:.3e}")
    if dtype == "float32":
        one = run(make_engine(name, dtype, max_tokens=need))
        for rid, rows in rp.logits.items():
            for p, row in rows.items():
                ref = one.logits[rid][p]
                assert float((row - ref).abs().max()) <= 2e-6 * float(ref.abs().max()), (rid, p)


@pytest.mark.parametrize("name,dtype", [(n, d) for n in ("A", "B", "R2") for d in ("float32", "bfloat16")]
                         + [("C", "bfloat16")])
def test_prompt_tokens_on_top_of_a_cache_that_is_not_empty(name, dtype):
    """A request brings many tokens at a position other than zero, beside a request that brings one; then the
    other way round; then one token each.  (The prefill kernels read earlier keys from the cache.)"""
    big = name == "C"
    first, more, again = (150, 200, 70) if big else (40, 50, 30)
    V = vocab(name)
    a = tiny.random_tokens(first + more + 1 + 1, V, 41)
    b = tiny.random_tokens(7 + 1 + again + 1, V, 42)
    e = make_engine(name, dtype, max_tokens=1024)
    rp = Replay(e)
    rp.step([("a", a[:first], [first - 1]), ("b", b[:7], [0, 6])])
    rp.step([("a", a[first:first + more], list(range(more))), ("b", [b[7]], [0])])
    rp.step([("a", [a[first + more]], [0]), ("b", b[8:8 + again], sparse_want(again))])
    rp.step([("a", [a[first + more + 1]], [0]), ("b", [b[8 + again]], [0])])
    rp.end("a")
    rp.end("b")
    e.check_device_errors()
    e.cache.check_consistency()
    worst = compare_with_plain(model_dir(name), {"a": a, "b": b}, rp, dtype)
    print(f"prompt on a cache, {name} {dtype}: worst relative error {worst:.3e}")


LONG_HEADS_OF_128 = {
    "architectures": ["Llama4ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 512,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 512,
    "num_local_experts": 4, "num_experts_per_tok": 1, "vocab_size": 1024, "nope_layer_interval": 2,
    "attention_chunk_size": 8192, "floor_scale": 8192, "attn_scale": 0.1, "initializer_range": 0.05,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_chunk_boundary_of_8192_against_plain(dtype):
    """Head size 128, chunk 8192 and temperature floor 8192, as in the benchmark's configuration: a prompt of
    9,000 tokens as two pieces whose cut (at 5,000) lies inside the first chunk, with rows on both sides of the
    chunk boundary, and decoding from 8,150 across position 8,192: all against the plain implementation."""
    from cpi_b200.engine import Engine
    d = tiny.make_model_dir(LONG_HEADS_OF_128, seed=4)
    try:
        long_prompt = tiny.random_tokens(9000, 1024, 1)
        dec = tiny.random_tokens(8150 + 60, 1024, 2)
        e = Engine.from_model_dir(d, dtype=dtype, max_tokens=9216, max_seqs=1, max_seq_len=9216,
                                  max_step_tokens=5000)
        rp = Replay(e)
        rows = [0, 4999, 5000, 8190, 8191, 8192, 8193, 8999]
        rp.step([("long", long_prompt, rows)])
        rp.end("long")
        rp.step([("dec", dec[:8150], [8149])])
        for t in dec[8150:]:
            rp.step([("dec", [t], [0])])
        rp.end("dec")
        e.check_device_errors()
        e.cache.check_consistency()
        worst = compare_with_plain(d, {"long": long_prompt, "dec": dec}, rp, dtype)
        print(f"chunk boundary 8192, {dtype}: worst relative error {worst:.3e}")
    finally:
        shutil.rmtree(d, ignore_errors=True)


SCOUT_TWO_LAYERS = {
    "architectures": ["Llama4ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 5120,
    "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192,
    "intermediate_size_mlp": 16384, "num_local_experts": 3, "num_experts_per_tok": 1,
    "interleave_moe_layer_step": 1, "vocab_size": 20011, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "nope_layer_interval": 2, "attention_chunk_size": 8192, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 8192, "attn_scale": 0.1,
    "tie_word_embeddings": False, "initializer_range": 0.02,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scout_layer_sizes_through_the_three_schedules(dtype):
    """The benchmark's layer sizes (width 5120, 40 / 8 heads of 128, experts of 8192) in two layers: each request
    whole and alone, with its last 32 tokens one by one, and in three unequal batches that follow one another in
    a cache sized for one of them."""
    from cpi_b200.engine import Engine
    V = SCOUT_TWO_LAYERS["vocab_size"]
    if "scout" not in _dirs:
        _dirs["scout"] = tiny.make_model_dir(SCOUT_TWO_LAYERS, seed=11)
    d = _dirs["scout"]
    try:
        shapes = [(70, 6), (33, 3), (5, 6), (129, 2)]
        need = sum(-(-(p + n) // 64) * 64 for p, n in shapes)
        e = Engine.from_model_dir(d, dtype=dtype, max_tokens=need)
        whole = {f"w{n}": tiny.random_tokens(n, V, 300 + n) for n in (1, 70, 131)}
        rp = Replay(e)
        run_whole(rp, whole)
        worst = compare_with_plain(d, whole, rp, dtype)
        tail = {f"t{n}": tiny.random_tokens(n, V, 400 + n) for n in (33, 100)}
        rp = Replay(e)
        pos = run_tail(rp, tail)
        worst = max(worst, compare_with_plain(d, tail, rp, dtype, pos))
        rp = Replay(e)
        batches, allreq = [], {}
        for b in range(3):
            reqs = {f"b{b}_{i}": (tiny.random_tokens(p + n, V, 1000 * b + 10 * i + p), p)
                    for i, (p, n) in enumerate(shapes)}
            batches.append(reqs)
            allreq.update({rid: t for rid, (t, p) in reqs.items()})
        pos = run_batched(rp, batches)
        worst = max(worst, compare_with_plain(d, allreq, rp, dtype, pos))
        e.check_device_errors()
        print(f"scout layer sizes, three schedules, {dtype}: worst relative error {worst:.3e}")
        del e
    finally:
        if dtype == "bfloat16":
            shutil.rmtree(_dirs.pop("scout"), ignore_errors=True)


@pytest.mark.parametrize("name,dtype,seed", [("A", "float32", 0), ("B", "float32", 1), ("B", "bfloat16", 2),
                                             ("R2", "float32", 3), ("C", "bfloat16", 4), ("C", "bfloat16", 5)])
def test_drawn_schedules_against_plain(name, dtype, seed):
    """Schedules drawn from a seed: batches of one to four requests with drawn prompt lengths (a single token
    among them), drawn places at which logits are wanted, a drawn number of decoded tokens per request so that
    requests leave the batch at drawn times, and `max_step_tokens` by turns absent, 37, 64 and 129; a cache that holds little more than
    the largest batch, so that pages and slots go round.  Every recorded row against the plain implementation."""
    import random
    rng = random.Random(1000 + seed)
    longest = 400 if name == "C" else 150
    V = vocab(name)
    batches = []
    for b in range(4):
        reqs = {}
        for i in range(rng.randint(1, 4)):
            p = 1 if rng.random() < 0.15 else rng.randint(2, longest)
            d = rng.randint(0, 10)
            reqs[f"b{b}r{i}"] = (tiny.random_tokens(p + d, V, 7000 + 97 * seed + 11 * b + i), p)
        batches.append(reqs)
    need = max(sum(-(-len(t) // 64) * 64 for t, _ in reqs.values()) for reqs in batches)
    cap = (None, 37, 64, 129)[seed % 4]
    e = make_engine(name, dtype, max_seqs=4, max_tokens=need, **({"max_step_tokens": cap} if cap else {}))
    rp = Replay(e)
    positions = {}
    for reqs in batches:
        items = []
        for rid, (t, p) in reqs.items():
            want = sorted({p - 1} | {rng.randrange(p) for _ in range(rng.randint(0, 6))})
            items.append((rid, t[:p], want))
            positions[rid] = list(want)
        rp.step(items)
        live, step = dict(reqs), 0
        while live:
            for rid in [r for r, (t, p) in live.items() if p + step >= len(t)]:
                rp.end(rid)
                del live[rid]
            if not live:
                break
            rp.step([(rid, [t[p + step]], [0]) for rid, (t, p) in live.items()])
            for rid, (t, p) in live.items():
                positions[rid].append(p + step)
            step += 1
        e.cache.check_consistency()
        assert e.cache.free_slots == e.cache.max_slots
    e.check_device_errors()
    all_reqs = {rid: t for reqs in batches for rid, (t, p) in reqs.items()}
    worst = compare_with_plain(model_dir(name), all_reqs, rp, dtype, positions)
    print(f"drawn schedule {seed} ({name} {dtype}, pieces of {cap}): {len(all_reqs)} requests, "
          f"worst relative error {worst:.3e}")
