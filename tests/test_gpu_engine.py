"""Engine against the plain implementation on a GPU: whole prompts, token-by-token tails, unequal batches."""
import pytest
import torch

import tiny
from helpers import Replay, compare_with_plain, tolerances

pytestmark = pytest.mark.gpu

_dirs, _engines = {}, {}


def model_dir(name):
    if name not in _dirs:
        _dirs[name] = tiny.make_model_dir(name)
    return _dirs[name]


def engine(name, dtype, max_tokens=1024):
    from cpi_b200.engine import Engine
    key = (name, dtype, max_tokens)
    if key not in _engines:
        _engines[key] = Engine.from_model_dir(model_dir(name), dtype=dtype, max_tokens=max_tokens)
    e = _engines[key]
    assert e.use_graphs, "every part of the library's own model is safe to capture"
    assert not e.cache.live_slots(), "a previous test left slots behind"
    return e


def vocab(name):
    c = tiny.config(name)
    return c.get("text_config", c)["vocab_size"]


# R2 lies inside what the reference's own engine computes: the plain implementation is checked against that engine at
# this point (tests/test_plain.py), so these cases tie the kernels to the reference's code and not only to its formulas
CASES = [(n, d) for n in ("A", "B", "R2") for d in ("float32", "bfloat16")] + [("C", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_each_alone(name, dtype):
    e = engine(name, dtype)
    lengths = (1, 64, 129, 400) if name == "C" else (1, 5, 33, 70, 150)
    reqs = {f"r{n}": tiny.random_tokens(n, vocab(name), 100 + n) for n in lengths}
    rp = Replay(e)
    for rid, toks in reqs.items():
        rp.step([(rid, toks, list(range(len(toks))))])
        rp.end(rid)
    worst = compare_with_plain(model_dir(name), reqs, rp, dtype)
    print(f"whole {name} {dtype}: worst relative error {worst:.3e}")
    e.cache.check_consistency()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(name, dtype):
    e = engine(name, dtype)
    reqs = {f"r{n}": tiny.random_tokens(n, vocab(name), 200 + n) for n in ((33, 170, 340) if name == "C" else (33, 70, 131))}
    rp = Replay(e)
    for rid, toks in reqs.items():
        n = len(toks)
        head = n - 32
        rp.step([(rid, toks[:head], [head - 1])])
        for i in range(head, n):
            rp.step([(rid, [toks[i]], [0])])
        rp.end(rid)
    positions = {rid: list(range(len(t) - 33, len(t))) for rid, t in reqs.items()}
    worst = compare_with_plain(model_dir(name), reqs, rp, dtype, positions)
    print(f"tail32 {name} {dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_one_after_another(name, dtype):
    """Batches of unequal prompts whose shorter requests end earlier; the cache is sized for one batch,
    so the second and third batch run in slots and pages that the first one gave back."""
    shapes = {"A": [(5, 24), (17, 9), (40, 24)], "B": [(1, 16), (9, 3), (33, 16), (70, 7)],
              "C": [(150, 20), (3, 8), (260, 20), (64, 1)], "R2": [(7, 12), (29, 5), (50, 18)]}[name]
    need = sum(-(-(p + d) // 64) * 64 for p, d in shapes)
    e = engine(name, dtype, max_tokens=need)
    all_reqs = {}
    rp = Replay(e)
    for b in range(3):
        reqs = {f"b{b}_{i}": tiny.random_tokens(p + d, vocab(name), 1000 * b + 10 * i + p)
                for i, (p, d) in enumerate(shapes)}
        all_reqs.update(reqs)
        prompt_len = {f"b{b}_{i}": p for i, (p, d) in enumerate(shapes)}
        rp.step([(rid, t[:prompt_len[rid]], [prompt_len[rid] - 1]) for rid, t in reqs.items()])
        live = dict(reqs)
        step = 0
        while live:
            for rid in [r for r, t in live.items() if prompt_len[r] + step >= len(t)]:
                rp.end(rid)
                del live[rid]
            if not live:
                break
            rp.step([(rid, [t[prompt_len[rid] + step]], [0]) for rid, t in live.items()])
            step += 1
        e.cache.check_consistency()
        assert e.cache.free_slots == e.cache.max_slots
    positions = {}
    for rid, t in all_reqs.items():
        i = int(rid.split("_")[1])
        positions[rid] = list(range(shapes[i][0] - 1, len(t)))
    worst = compare_with_plain(model_dir(name), all_reqs, rp, dtype, positions)
    print(f"batched {name} {dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_cuts_agree_bitwise_in_float32(name):
    """The same position gives the same logits whole, token by token, and inside a batch."""
    e = engine(name, "float32")
    V = vocab(name)
    a, b = tiny.random_tokens(50, V, 1), tiny.random_tokens(21, V, 2)
    rp = Replay(e)
    rp.step([("whole", a, [49])]); rp.end("whole")
    rp.step([("cut", a[:30], [])])
    for i in range(30, 50):
        rp.step([("cut", [a[i]], [0])])
    rp.end("cut")
    rp.step([("other", b[:20], [19]), ("batched", a[:49], [48])])
    rp.step([("other", [b[20]], [0]), ("batched", [a[49]], [0])])
    rp.end("other"); rp.end("batched")
    w, c, bt = rp.logits["whole"][49], rp.logits["cut"][49], rp.logits["batched"][49]
    scale = float(w.abs().max())
    assert float((w - c).abs().max()) <= 2e-6 * scale
    assert float((w - bt).abs().max()) <= 2e-6 * scale


@pytest.mark.parametrize("name,dtype,prompt,steps", [("A", "float32", 7, 300), ("C", "bfloat16", 100, 420),
                                                      ("B", "bfloat16", 3, 150)])
def test_long_decoding(name, dtype, prompt, steps):
    """Hundreds of single-token steps (through the captured decode graph), across page, chunk and
    temperature-floor boundaries, in a batch with a second, shorter request that ends on the way."""
    n = prompt + steps
    e = engine(name, dtype, max_tokens=1024)
    a, b = tiny.random_tokens(n, vocab(name), 31), tiny.random_tokens(prompt + 40, vocab(name), 32)
    rp = Replay(e)
    rp.step([("a", a[:prompt], [prompt - 1]), ("b", b[:prompt], [prompt - 1])])
    for i in range(prompt, n):
        items = [("a", [a[i]], [0])]
        if i < len(b):
            items.append(("b", [b[i]], [0]))
        rp.step(items)
        if i == len(b) - 1:
            rp.end("b")
    rp.end("a")
    checks = sorted(set(range(prompt - 1, n, 7)) | {n - 1, n - 2})
    worst = compare_with_plain(model_dir(name), {"a": a, "b": b}, rp, dtype,
                               {"a": checks, "b": list(range(prompt - 1, len(b), 5))})
    print(f"long decoding {name} {dtype}: worst relative error {worst:.3e}")
    # the same steps once more without the recording: decode now replays captured graphs, and must give
    # the very same bits as the eager launches above
    from cpi_b200.engine import StepEntry
    e.capture_routing(False)
    assert e.use_graphs
    sa, sb = e.acquire_slot(), e.acquire_slot()
    replays_before = e.graph_kernel_launches
    e.step([StepEntry(sa, a[:prompt], []), StepEntry(sb, b[:prompt], [])])
    for i in range(prompt, n):
        entries = [StepEntry(sa, [a[i]], [0])]
        if i < len(b):
            entries.append(StepEntry(sb, [b[i]], [0]))
        out = e.step(entries).cpu()
        if i in checks:
            assert torch.equal(out[0], rp.logits["a"][i]), f"graph replay differs from eager at position {i}"
        if i == len(b) - 1:
            e.release_slot(sb)
    e.release_slot(sa)
    e.check_device_errors()
    assert e.graph_kernel_launches > replays_before


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype):
    """Positions 0, 1, 2: as a three-token prompt, and one by one from an empty cache."""
    e = engine(name, dtype)
    t = tiny.random_tokens(3, vocab(name), 77)
    rp = Replay(e)
    rp.step([("whole", t, [0, 1, 2])]); rp.end("whole")
    for i in range(3):
        rp.step([("single", [t[i]], [0])])
    rp.end("single")
    compare_with_plain(model_dir(name), {"whole": t, "single": t}, rp, dtype)


def test_random_weights_drawn_on_the_gpu_equal_the_folder_written_on_the_cpu():
    """The generator is counter based: the same (seed, name, element) gives the same bits on both devices, so a
    model drawn in place and one read from its folder give the same logits bit for bit."""
    from cpi_b200.engine import Engine
    from cpi_b200.engine.model import tensor_requirements
    from cpi_b200.weights.random_init import RandomSource
    cfg, seed = tiny.config("B"), 11
    a = Engine.from_random(cfg, seed=seed, dtype="bfloat16", max_tokens=256)
    b = Engine.from_model_dir(tiny.make_model_dir("B", seed=seed), dtype="bfloat16", max_tokens=256)
    src = RandomSource(tensor_requirements(a.spec), seed, a.spec.initializer_range)
    for n in src.names():
        assert torch.equal(src.get(n, "cuda").cpu(), src.get(n, "cpu")), n
    t = tiny.random_tokens(40, a.spec.vocab_size, 3)
    outs = []
    for e in (a, b):
        rp = Replay(e)
        rp.step([("x", t, [len(t) - 1])])
        outs.append(rp.logits["x"][len(t) - 1])
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_stored_in_float32_stay_float32(dtype):
    """A model folder whose tensors are F32: they are kept in 32-bit, and both precisions still match."""
    from cpi_b200.engine import Engine
    d = tiny.make_model_dir("B", seed=5, dtype=torch.float32)
    e = Engine.from_model_dir(d, dtype=dtype, max_tokens=256)
    assert e.model.layers[1].mixer.w_qkv.dtype == torch.float32 and e.model.embedding.dtype == torch.float32
    reqs = {"x": tiny.random_tokens(50, 1000, 8), "y": tiny.random_tokens(9, 1000, 9)}
    rp = Replay(e)
    rp.step([("x", reqs["x"][:40], [39]), ("y", reqs["y"][:8], [7])])
    rp.step([("x", [reqs["x"][40]], [0]), ("y", [reqs["y"][8]], [0])])
    rp.end("y")
    for t in reqs["x"][41:]:
        rp.step([("x", [t], [0])])
    rp.end("x")
    compare_with_plain(d, reqs, rp, dtype, {"x": list(range(39, 50)), "y": [7, 8]})


def test_long_context_across_the_chunk_boundary_both_kernel_families_agree():
    """Head size 128, chunk 8192, temperature floor 8192: a 9,000-token prompt (its tiles straddle the
    chunk boundary and run as two pieces) and decoding from 8,150 across position 8,192, once on the
    tensor-core kernels and once on the general ones.  With one expert per token a near-tie of two router
    logits can fall either way in bfloat16, and then the row is another function of its input: rows whose
    expert choices differ between the two runs are set aside (they must be few; that such choices are
    near-ties is checked against the plain router in the other tests)."""
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.parts import attention, linear
    cfg = {
        "architectures": ["Llama4ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 512,
        "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 512,
        "num_local_experts": 4, "num_experts_per_tok": 1, "vocab_size": 1024, "nope_layer_interval": 2,
        "attention_chunk_size": 8192, "floor_scale": 8192, "attn_scale": 0.1, "initializer_range": 0.05,
        "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
    }
    d = tiny.make_model_dir(cfg, seed=4)
    long_prompt = tiny.random_tokens(9000, 1024, 1)
    dec = tiny.random_tokens(8150 + 120, 1024, 2)
    outs = {}
    for fast in (True, False):
        attention.use_tensor_core_kernels = fast
        linear.use_tensor_cores = fast
        try:
            e = Engine.from_model_dir(d, dtype="bfloat16", max_tokens=9216 + 8320, max_seqs=2, max_seq_len=9216)
            cap = e.capture_routing(True)
            chosen = lambda: torch.cat([torch.cat([x.cpu() for x in cap[l]]) for l in sorted(cap)], 1)
            s = e.acquire_slot()
            rows = [e.step([StepEntry(s, long_prompt, [8191, 8192, 8999])]).float().cpu()]
            experts = [chosen()[[8191, 8192, 8999]]]
            e.release_slot(s)
            s = e.acquire_slot()
            e.step([StepEntry(s, dec[:8150], [])])
            for t in dec[8150:]:
                for lst in cap.values():
                    lst.clear()
                rows.append(e.step([StepEntry(s, [t], [0])]).float().cpu())
                experts.append(chosen())
            e.release_slot(s)
            e.check_device_errors()
            e.cache.check_consistency()
            outs[fast] = (torch.cat(rows), torch.cat(experts))
            del e
        finally:
            attention.use_tensor_core_kernels = True
            linear.use_tensor_cores = True
    (a, ea), (b, eb) = outs[True], outs[False]
    same = (ea == eb).all(-1)
    assert float(same.float().mean()) >= 0.95, f"{int((~same).sum())} of {len(same)} rows chose other experts"
    a, b = a[same], b[same]
    scale = float(b.abs().max())
    err = float((a - b).abs().max()) / scale
    print(f"long context: tensor-core vs general kernels, worst relative difference {err:.3e} "
          f"({int((~same).sum())} rows with other experts set aside)")
    assert err <= 3e-2
    assert float((a.argmax(-1) == b.argmax(-1)).float().mean()) > 0.9


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


@pytest.mark.parametrize("which", ["C", "scout"])
def test_bfloat16_drift_against_float32(which):
    """The reference's measure of a reduced-precision path (tools/moe_cuda_bench.py:177-212): is the best token
    the same, how many of the five best tokens are shared, mean and largest absolute difference -- of the
    bfloat16 path against the float32 path on the same weights, prompt rows and decoded rows.  Rows where the
    two precisions chose other experts (near-ties of the router, checked against the plain router elsewhere)
    are counted and set aside."""
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.engine.drift import compare_logits
    if which == "scout":
        if "scout" not in _dirs:
            _dirs["scout"] = tiny.make_model_dir(SCOUT_TWO_LAYERS, seed=11)
        d, vocab = _dirs["scout"], SCOUT_TWO_LAYERS["vocab_size"]
    else:
        d, vocab = model_dir("C"), 777
    prompt, more = tiny.random_tokens(150, vocab, 21), tiny.random_tokens(24, vocab, 22)
    rows, experts = {}, {}
    for dtype in ("float32", "bfloat16"):
        e = Engine.from_model_dir(d, dtype=dtype, max_tokens=256)
        cap = e.capture_routing(True)
        chosen = lambda: torch.cat([torch.cat([x.cpu() for x in cap[l]]) for l in sorted(cap)], 1)
        s = e.acquire_slot()
        out = [e.step([StepEntry(s, prompt, list(range(len(prompt))))]).float().cpu()]
        ex = [chosen()]
        for t in more:
            for lst in cap.values():
                lst.clear()
            out.append(e.step([StepEntry(s, [t], [0])]).float().cpu())
            ex.append(chosen())
        e.release_slot(s)
        e.check_device_errors()
        rows[dtype], experts[dtype] = torch.cat(out), torch.cat(ex)
        del e
    same = (experts["float32"] == experts["bfloat16"]).all(-1)
    flipped = (~same).nonzero().flatten().tolist()
    # a position whose expert differs has other keys and values in the layers above, so the rows after it in the
    # sequence differ by more than rounding too (measured: twice the typical row): the figures are taken of the
    # rows before the first such position
    clean = flipped[0] if flipped else len(same)
    assert clean >= 40 and len(flipped) <= 0.1 * len(same), flipped
    m = compare_logits(rows["float32"][:clean], rows["bfloat16"][:clean], 5)
    print(f"bfloat16 against float32 ({which}): rows {flipped} of {len(same)} chose other experts; of the {clean} rows "
          f"before them: best token the same in {m['top1_match']:.3f}, five best shared {m['overlap_at_k']:.3f}, "
          f"mean |d| {m['mean_abs']:.3e}, max |d| {m['max_abs']:.3e}; logits: spread {m['ref_std']:.3e}, "
          f"largest {m['ref_max_abs']:.3e}")
    assert m["max_abs"] <= tolerances("bfloat16")[0] * m["ref_max_abs"]       # the suite's bound for a bfloat16 row
    assert m["mean_abs"] <= 0.02 * m["ref_std"]
    assert m["top1_match"] >= 0.9 and m["overlap_at_k"] >= 0.9
    if which == "scout":
        import shutil
        shutil.rmtree(_dirs.pop("scout"), ignore_errors=True)
