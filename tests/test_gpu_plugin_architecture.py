"""A whole architecture from outside the package: a module that this test writes into a temporary folder registers
a block arrangement and an architecture, the environment variable CPI_B200_PLUGINS names it, and from then on the
library's own programs know it by its config.json name.  The toy has what Llama4 has not: layers whose attention
sees a sliding window of positions (a third kind of cache group), a block whose feed-forward reads the layer's
input instead of the mixer's output, and no experts.  It goes the whole way: random-weights folder, `bin/trace_run`
in a process of its own (each request whole, then in a batch with the last tokens one by one, in both precisions),
and greedy generation through `Model`, each against a plain implementation written here from the plain parts."""
import math
import os
import subprocess
import sys
import tempfile
import textwrap

import pytest
import torch

import plain_llama4 as P
import tiny
from helpers import TraceOutput

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PLUGIN = textwrap.dedent('''
    """A toy architecture registered from outside the package."""
    from dataclasses import dataclass

    from cpi_b200.config.common import ConfigError
    from cpi_b200.config.registry import Architecture, register_architecture
    from cpi_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
    from cpi_b200.parts import Block, register_block


    @register_block("toy_parallel")
    class ParallelBlock(Block):
        """x += mixer(norm1(x)) + feed_forward(norm2(x)): the feed-forward reads the layer's input, not the
        mixer's output."""
        graph_safe = True

        def __init__(self, spec, prefix="", **_):
            super().__init__(spec, prefix)

        def run(self, layer, residual, batch, cache):
            h = layer.mixer_norm(residual, batch.dtype)
            h2 = layer.feed_forward_norm(residual, batch.dtype)
            layer.mixer.forward(h, residual, batch, cache)
            layer.feed_forward.forward(h2, residual, batch)


    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        num_hidden_layers: int
        vocab_size: int
        intermediate_size: int
        num_attention_heads: int
        num_key_value_heads: int
        head_dim: int
        rms_norm_eps: float
        rope_theta: float
        sliding_window: int
        layer_types: tuple

        @staticmethod
        def from_json_dict(raw):
            keys = ToyConfig.__dataclass_fields__
            missing = [k for k in keys if k not in raw]
            if missing:
                raise ConfigError("config.json: missing " + ", ".join(missing))
            c = ToyConfig(**{k: (tuple(raw[k]) if k == "layer_types" else raw[k]) for k in keys})
            if len(c.layer_types) != c.num_hidden_layers or any(t not in ("sliding", "full") for t in c.layer_types):
                raise ConfigError("config.json: layer_types must name 'sliding' or 'full' for every layer")
            return c


    def build_spec(c):
        norm = {"size": c.hidden_size, "eps": float(c.rms_norm_eps)}
        layers = []
        for i, kind in enumerate(c.layer_types):
            window = {"kind": "sliding", "size": c.sliding_window} if kind == "sliding" else {"kind": "full", "size": 0}
            mixer = PartSpec("attention", {
                "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
                "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                "softmax_scale": float(c.head_dim) ** -0.5,
                "position": PartSpec("rope", {"head_dim": c.head_dim, "theta": float(c.rope_theta),
                                              "pairing": "half_split", "scaling": None}),
                "qk_norm": False, "qk_norm_eps": float(c.rms_norm_eps), "qk_norm_order": "after_rope",
                "window": window, "query_temperature": None})
            layers.append(LayerSpec(
                prefix=f"blocks.{i}.", block=PartSpec("toy_parallel", {}), mixer=mixer,
                feed_forward=PartSpec("dense_swiglu", {"hidden_size": c.hidden_size,
                                                       "intermediate_size": c.intermediate_size}),
                mixer_norm=PartSpec("rmsnorm", {**norm, "weight": "norm1.weight"}),
                feed_forward_norm=PartSpec("rmsnorm", {**norm, "weight": "norm2.weight"})))
        return ModelSpec(
            architecture="ToySlidingForCausalLM", hidden_size=c.hidden_size, vocab_size=c.vocab_size,
            embedding=PartSpec("token_embedding", {"weight": "wte.weight", "vocab_size": c.vocab_size,
                                                   "hidden_size": c.hidden_size}),
            layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(c.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {**norm, "weight": "final_norm.weight"}),
            head=PartSpec("linear_head", {"weight": "wte.weight", "vocab_size": c.vocab_size,
                                          "hidden_size": c.hidden_size}),
            initializer_range=0.08)


    register_architecture(Architecture("ToySlidingForCausalLM", ToyConfig.from_json_dict, build_spec))
''')

# two configurations that differ in every size: one for the general kernels' head size, one whose head size and
# widths let the bfloat16 path take the tensor-core products and both tensor-core attention kernels
CONFIGS = {
    "small": dict(hidden_size=72, num_hidden_layers=3, vocab_size=211, intermediate_size=100, num_attention_heads=6,
                  num_key_value_heads=3, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0, sliding_window=23,
                  layer_types=["sliding", "full", "sliding"]),
    "wide": dict(hidden_size=128, num_hidden_layers=2, vocab_size=307, intermediate_size=136, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=50000.0, sliding_window=150,
                 layer_types=["full", "sliding"]),
}


@pytest.fixture(scope="module")
def plugin_dir():
    d = tempfile.mkdtemp(prefix="cpi_b200_plugin_")
    with open(os.path.join(d, "toy_sliding_arch.py"), "w") as f:
        f.write(PLUGIN)
    old_path, old_env = list(sys.path), os.environ.get("CPI_B200_PLUGINS")
    sys.path.insert(0, d)
    os.environ["CPI_B200_PLUGINS"] = "toy_sliding_arch"
    import importlib
    importlib.import_module("toy_sliding_arch")          # this process may have loaded the registry already
    yield d
    sys.path[:] = old_path
    if old_env is None:
        os.environ.pop("CPI_B200_PLUGINS", None)
    else:
        os.environ["CPI_B200_PLUGINS"] = old_env


def model_dir(plugin_dir, name):
    from cpi_b200.weights.random_init import write_random_model
    d = os.path.join(plugin_dir, "model_" + name)
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        write_random_model(d, dict(CONFIGS[name], architectures=["ToySlidingForCausalLM"]), seed=11)
    return d


def plain_forward(c, W, tokens):
    """Logits [n, V] of the toy, from the plain parts."""
    n = len(tokens)
    pos = list(range(n))
    NH, NKV, D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    fr = P.rope_frequencies({"head_dim": D, "rope_theta": c["rope_theta"], "rope_scaling": None})
    x = P.embedding(W["wte.weight"], tokens)
    p = torch.arange(n)
    for i, kind in enumerate(c["layer_types"]):
        pre = f"blocks.{i}."
        h = P.rmsnorm(x, W[pre + "norm1.weight"], c["rms_norm_eps"])
        h2 = P.rmsnorm(x, W[pre + "norm2.weight"], c["rms_norm_eps"])
        q = P.rope((h @ W[pre + "self_attn.q_proj.weight"].T).reshape(n, NH, D), pos, fr, "half_split")
        k = P.rope((h @ W[pre + "self_attn.k_proj.weight"].T).reshape(n, NKV, D), pos, fr, "half_split")
        v = (h @ W[pre + "self_attn.v_proj.weight"].T).reshape(n, NKV, D)
        mask = p[None, :] <= p[:, None]
        if kind == "sliding":
            mask &= p[None, :] > p[:, None] - c["sliding_window"]       # the last `sliding_window` positions
        a = P.attention(q, k, v, mask, 1.0 / math.sqrt(D)) @ W[pre + "self_attn.o_proj.weight"].T
        f = P.swiglu_mlp(h2, W[pre + "feed_forward.gate_proj.weight"], W[pre + "feed_forward.up_proj.weight"],
                         W[pre + "feed_forward.down_proj.weight"])
        x = x + a + f
    return P.rmsnorm(x, W["final_norm.weight"], c["rms_norm_eps"]) @ W["wte.weight"].T


@pytest.mark.parametrize("name,dtype", [("small", "float32"), ("small", "bfloat16"), ("wide", "float32"),
                                        ("wide", "bfloat16")])
def test_replay_tool_runs_an_architecture_from_a_plugin(plugin_dir, name, dtype):
    d = model_dir(plugin_dir, name)
    c, W = CONFIGS[name], P.read_weights(d)
    lengths = (3, 70, 41) if name == "small" else (190, 9, 333)         # past the window in both
    reqs = {f"r{i}": tiny.random_tokens(n, c["vocab_size"], 900 + n) for i, n in enumerate(lengths)}
    trace = os.path.join(plugin_dir, f"trace_{name}.txt")
    with open(trace, "w") as f:
        for rid, t in reqs.items():
            f.write(rid + ": " + " ".join(map(str, t)) + "\n")
    env = dict(os.environ, CPI_B200_PLUGINS="toy_sliding_arch",
               PYTHONPATH=plugin_dir + os.pathsep + os.environ.get("PYTHONPATH", ""))
    tol = 2e-5 if dtype == "float32" else 2e-2
    # whole; as one batch with the last two tokens one by one; each alone with its last 60 tokens one by one (the
    # longer requests then decode far past the window, and the window's group gives pages back as they go)
    for mode, tail in (("whole", 2), ("batched", 2), ("tail32", 60)):
        out = os.path.join(plugin_dir, f"out_{name}_{dtype}_{mode}")
        need = sum(-(-len(t) // 64) * 64 for t in reqs.values())
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                            "--out", out, "--max-tokens", str(need), "--trace", trace, "--mode", mode,
                            "--batch-size", "3", "--tail", str(tail)], env=env, capture_output=True, text=True,
                           timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        got = TraceOutput(out)
        worst = 0.0
        for rid, t in reqs.items():
            ref = plain_forward(c, W, t)
            rows = got.logits[rid]
            assert rows, rid
            if mode == "whole":
                assert sorted(rows) == list(range(len(t)))
            scale = float(ref.abs().max())
            for p_, row in rows.items():
                err = float((row - ref[p_]).abs().max()) / scale
                worst = max(worst, err)
                assert err <= tol, (name, dtype, mode, rid, p_, err)
        print(f"plugin architecture {name} {dtype} {mode}: worst relative error {worst:.3e}")
    # without the variable the same folder is refused by name
    env.pop("CPI_B200_PLUGINS")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                        "--out", os.path.join(plugin_dir, "out_refused"), "--max-tokens", "64"], env=env,
                       input="", capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "ToySlidingForCausalLM" in r.stderr and "not registered" in r.stderr


@pytest.mark.parametrize("name,dtype", [("small", "float32"), ("wide", "bfloat16")])
def test_generation_with_an_architecture_from_a_plugin(plugin_dir, name, dtype):
    from cpi_b200.api import Model
    d = model_dir(plugin_dir, name)
    c, W = CONFIGS[name], P.read_weights(d)
    lengths = (30, 5, 61) if name == "small" else (170, 40, 8)
    prompts = [tiny.random_tokens(n, c["vocab_size"], 60 + n) for n in lengths]
    m = Model.load(d, dtype=dtype, max_batch=2, max_context=256)           # three requests in two slots
    groups = {(g.req.window_kind, g.req.window_size) for g in m.engine.cache.groups}
    assert groups == {("sliding", c["sliding_window"]), ("full", 0)}
    got = m.generate(prompts, max_new=8, temperature=0.0, stop_ids=[])
    tol = 2e-5 if dtype == "float32" else 4e-2
    for p_, g in zip(prompts, got):
        seq = list(p_)
        assert len(g.tokens) == 8
        for tok in g.tokens:
            lg = plain_forward(c, W, seq)[-1]
            best = int(torch.argmax(lg))
            if tok != best:
                assert float(lg[best] - lg[tok]) <= tol * float(lg.abs().max()), (name, dtype, len(seq), tok, best)
            seq.append(tok)
    m.engine.check_device_errors()
    m.engine.cache.check_consistency()
    assert m.engine.cache.free_slots == m.engine.cache.max_slots
