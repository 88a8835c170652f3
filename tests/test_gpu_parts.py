"""Each part alone against the plain implementation's function for it; the run order as data; and a toy
mixer with state of its own, defined here, registered and stepped without a change to the library."""
import dataclasses

import pytest
import torch

import plain_llama4 as P
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _llama4(name):
    from cpi_b200.config import spec_from_model_dir
    d = tiny.make_model_dir(name)
    cfg, spec = spec_from_model_dir(d)
    return d, spec, P.read_config(d), P.read_weights(d)


def _source(d):
    from cpi_b200.weights import SafetensorsSource
    return SafetensorsSource(d)


def _batch(seqs, dtype):
    """seqs: list of (slot, start, n)."""
    from cpi_b200.engine.batch import BatchStager
    st = BatchStager(DEV)
    return st.stage([s for s, _, _ in seqs], [a for _, a, _ in seqs], [[0] * n for _, _, n in seqs],
                    [[] for _ in seqs], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from cpi_b200.config import PartSpec
    from cpi_b200.parts import Workspace, build_part
    from cpi_b200.weights import DictSource
    w = torch.randn(100).bfloat16()
    n = build_part("norm", PartSpec("rmsnorm", {"size": 100, "eps": 1e-6, "weight": "n.weight"}), "x.",
                   workspace=Workspace(DEV), tag="t")
    assert [r.name for r in n.requirements()] == ["x.n.weight"] and n.requirements()[0].init == "ones"
    n.load(DictSource({"x.n.weight": w}), DEV)
    x = torch.randn(9, 100, device=DEV)
    ref = P.rmsnorm(x.cpu(), w.float(), 1e-6)
    out = n(x, dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert out.dtype == dtype and float((out.float().cpu() - ref).abs().max()) <= tol * float(ref.abs().max())


def test_position_part_matches_plain_frequencies():
    from cpi_b200.parts import build_part
    d, spec, c, W = _llama4("A")
    pos = build_part("position", spec.layers[0].mixer["position"])
    assert (pos.frequencies == P.rope_frequencies(c)).all() and not pos.interleaved
    none = build_part("position", spec.layers[3].mixer["position"])
    assert none.encoding() is None
    pos.prepare(DEV)
    enc = pos.encoding()
    assert type(enc).__name__ == "RotaryEncoding" and not enc.interleaved
    assert (enc.inv_freq.cpu().numpy() == P.rope_frequencies(c)).all()
    d, spec, c, W = _llama4("B")
    posb = build_part("position", spec.layers[0].mixer["position"])
    assert (posb.frequencies == P.rope_frequencies(c)).all() and posb.interleaved


@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 3), ("B", 1), ("B", 2), ("C", 0), ("C", 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixer_alone(name, layer, dtype):
    """The mixer on a whole sequence, and again cut into a prefix and single tokens: both equal the plain part."""
    from cpi_b200.cache import CacheManager
    from cpi_b200.parts import CacheView, Workspace, build_part
    d, spec, c, W = _llama4(name)
    ls = spec.layers[layer]
    mixer = build_part("mixer", ls.mixer, ls.prefix, workspace=Workspace(DEV))
    mixer.load(_source(d), DEV)
    n, H = 150, spec.hidden_size
    h = (torch.randn(n, H, generator=torch.Generator().manual_seed(layer)) * 0.5)
    ref = P.attention_part(c, W, ls.prefix, layer, h.to(dtype).float(), list(range(n)))
    cache = CacheManager({0: mixer.kv_requirement()}, {}, max_tokens=512, dtype=dtype, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for cuts in ([n], [100] + [1] * 50):
        slot = cache.acquire()
        got = torch.zeros(n, H, device=DEV)
        off = 0
        for k in cuts:
            cache.prepare_step([slot], [k])
            b = _batch([(slot, off, k)], dtype)
            mixer.forward(h[off:off + k].to(dtype).to(DEV), got[off:off + k], b, CacheView(cache, 0))
            cache.commit_step([slot], [k])
            off += k
        err = float((got.cpu() - ref).abs().max()) / float(ref.abs().max())
        assert err <= tol, (cuts[:2], err)
        cache.release(slot)


@pytest.mark.parametrize("name,layer", [("A", 1), ("B", 0), ("B", 3), ("C", 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_alone(name, layer, dtype):
    from cpi_b200.parts import Workspace, build_part
    d, spec, c, W = _llama4(name)
    ls = spec.layers[layer]
    ff = build_part("feed_forward", ls.feed_forward, ls.prefix, workspace=Workspace(DEV))
    ff.load(_source(d), DEV)
    T, H = 37, spec.hidden_size
    h = torch.randn(T, H, generator=torch.Generator().manual_seed(3))
    hq = h.to(dtype)
    if hasattr(ff, "capture"):
        ff.capture = []
    got = torch.zeros(T, H, device=DEV)
    ff.forward(hq.to(DEV), got, _batch([(0, 0, T)], dtype))
    forced = ff.capture[0].cpu() if getattr(ff, "capture", None) else None
    ref, routing = P.feed_forward_part(c, W, ls.prefix, layer, hq.float(), forced)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((got.cpu() - ref).abs().max()) <= tol * float(ref.abs().max())
    if routing is not None:                 # the engine's choices are the plain router's, up to near-ties
        logits, own = routing
        k = c["num_experts_per_tok"]
        kth = torch.sort(logits, -1, descending=True).values[:, k - 1]
        gap = kth[:, None] - torch.gather(logits, 1, forced.long())
        assert float(gap.max()) <= (1e-5 if dtype == torch.float32 else 1e-2) * float(logits.abs().max())


def test_layer_named_twice_in_the_run_order_equals_a_model_with_the_layer_copied():
    """run_order (0, 0, 1): layer 0's weights are used twice, each use with a cache of its own."""
    from cpi_b200.config import RunEntry
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.weights import DictSource
    d, spec, c, W = _llama4("A")
    two = dataclasses.replace(spec, layers=spec.layers[:2], run_order=(RunEntry(0), RunEntry(0), RunEntry(1)))
    src = _source(d)
    keep = {n: src.get(n, "cpu") for n in src.names() if ".layers.2." not in n and ".layers.3." not in n}
    e = Engine(two, DictSource(keep), dtype="float32", max_tokens=256)
    assert sum(len(g.entries) for g in e.cache.groups) == 3
    toks = tiny.random_tokens(40, 512, 9)
    s = e.acquire_slot()
    got = e.step([StepEntry(s, toks, list(range(40)))]).cpu()
    e.release_slot(s)
    c3 = dict(c, num_hidden_layers=3, nope_layer_interval=0)
    W3 = dict(W)
    for k_, v in W.items():
        if ".layers.0." in k_:
            W3[k_.replace(".layers.0.", ".layers.1.")] = v
        if ".layers.1." in k_:
            W3[k_.replace(".layers.1.", ".layers.2.")] = v
    ref = P.forward(c3, W3, toks)
    assert float((got - ref).abs().max()) <= 2e-5 * float(ref.abs().max())


def test_an_entry_that_reads_another_entrys_cache():
    """run_order (0, 1 reading 0's cache): layer 1 keeps no keys of its own; cuts agree bitwise."""
    from cpi_b200.config import RunEntry
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.weights import DictSource
    d, spec, c, W = _llama4("A")
    sp = dataclasses.replace(spec, layers=spec.layers[:2], run_order=(RunEntry(0), RunEntry(1, cache_of=0)))
    src = _source(d)
    keep = {n: src.get(n, "cpu") for n in src.names() if ".layers.2." not in n and ".layers.3." not in n
            and ".layers.1.self_attn.k_proj" not in n and ".layers.1.self_attn.v_proj" not in n}
    e = Engine(sp, DictSource(keep), dtype="float32", max_tokens=256)     # layer 1 needs no k/v weights
    assert sum(len(g.entries) for g in e.cache.groups) == 1
    toks = tiny.random_tokens(45, 512, 4)
    s = e.acquire_slot()
    whole = e.step([StepEntry(s, toks, [44])]).cpu()
    e.release_slot(s)
    s = e.acquire_slot()
    e.step([StepEntry(s, toks[:30], [])])
    for t in toks[30:]:
        last = e.step([StepEntry(s, [t], [0])]).cpu()
    e.release_slot(s)
    assert torch.equal(whole, last)
    # it differs from the model whose second layer has keys of its own
    keep2 = {n: src.get(n, "cpu") for n in src.names() if ".layers.2." not in n and ".layers.3." not in n}
    own = Engine(dataclasses.replace(sp, run_order=(RunEntry(0), RunEntry(1))), DictSource(keep2), dtype="float32",
                 max_tokens=256)
    s = own.acquire_slot()
    other = own.step([StepEntry(s, toks, [44])]).cpu()
    assert float((other - whole).abs().max()) > 1e-4


# ---------------------------------------------------------------------------------------------- toy mixer
def _register_toy():
    """A mixer with fixed-size state: out_t = W * mean of the inputs up to t.  State: running sum and count."""
    from cpi_b200.cache import StateRequirement
    from cpi_b200.parts import Mixer, register_mixer
    from cpi_b200.weights import TensorReq

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
            super().__init__(spec, prefix)
            self.h = int(spec["hidden_size"])

        def requirements(self):
            return [TensorReq(self.prefix + "mix.weight", (self.h, self.h))]

        def load(self, source, device):
            self.w = source.get(self.prefix + "mix.weight", device).float()

        def state_requirements(self):
            return [StateRequirement("sum", (self.h,)), StateRequirement("count", (1,))]

        def forward(self, h, residual, batch, cache):
            total, count = cache.state("sum"), cache.state("count")
            off = 0
            for slot, n in zip(batch.slots, batch.n_new):          # a scan over the new tokens from the state
                x = h[off:off + n].float()
                run = total[slot] + torch.cumsum(x, 0)
                cnt = count[slot] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)[:, None]
                residual[off:off + n] += (run / cnt) @ self.w.T
                total[slot] = run[-1]
                count[slot] = cnt[-1]
                off += n

    return RunningMean


def test_toy_mixer_with_state_registers_builds_and_steps():
    from cpi_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.engine.model import tensor_requirements
    from cpi_b200.weights import DictSource, RandomSource
    _register_toy()
    H, V, I = 48, 90, 80
    norm = lambda w: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "weight": w})
    layers = tuple(LayerSpec(prefix=f"l{i}.", block=PartSpec("pre_norm"),
                             mixer=PartSpec("toy_running_mean", {"hidden_size": H}),
                             feed_forward=PartSpec("dense_swiglu", {"hidden_size": H, "intermediate_size": I}),
                             mixer_norm=norm("n1.weight"), feed_forward_norm=norm("n2.weight")) for i in range(2))
    spec = ModelSpec(architecture="Toy", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"weight": "emb.weight"}), layers=layers,
                     run_order=(RunEntry(0), RunEntry(1)), final_norm=norm("norm.weight"),
                     head=PartSpec("linear_head", {"weight": "emb.weight"}), initializer_range=0.1)
    reqs = tensor_requirements(spec)
    src = RandomSource(reqs, 3, 0.1)
    drawn = {n: src.get(n, "cpu") for n in src.names()}
    W = {n: t.float() for n, t in drawn.items()}
    e = Engine(spec, DictSource(drawn), dtype="float32", max_tokens=512)
    assert not e.cache.groups and len(e.cache.state) == 4          # no keys or values, two states per entry
    assert not e.use_graphs                  # the toy mixer reads host values of the step and does not claim otherwise

    def plain(tokens):
        x = W["emb.weight"][tokens]
        for i in range(2):
            h = P.rmsnorm(x, W[f"l{i}.n1.weight"], 1e-5)
            mean = torch.cumsum(h, 0) / torch.arange(1, len(tokens) + 1)[:, None]
            x = x + mean @ W[f"l{i}.mix.weight"].T
            h2 = P.rmsnorm(x, W[f"l{i}.n2.weight"], 1e-5)
            x = x + P.swiglu_mlp(h2, W[f"l{i}.feed_forward.gate_proj.weight"], W[f"l{i}.feed_forward.up_proj.weight"],
                                 W[f"l{i}.feed_forward.down_proj.weight"])
        return P.rmsnorm(x, W["norm.weight"], 1e-5) @ W["emb.weight"].T

    a, b = tiny.random_tokens(30, V, 1), tiny.random_tokens(11, V, 2)
    ra, rb = plain(a), plain(b)
    for round_ in range(2):                                         # the second round reuses the slots
        sa, sb = e.acquire_slot(), e.acquire_slot()
        out = e.step([StepEntry(sa, a[:25], [24]), StepEntry(sb, b[:9], [0, 8])]).cpu()
        rows = [(out[0], ra[24]), (out[1], rb[0]), (out[2], rb[8])]
        out = e.step([StepEntry(sa, [a[25]], [0]), StepEntry(sb, [b[9]], [0])]).cpu()
        rows += [(out[0], ra[25]), (out[1], rb[9])]
        e.release_slot(sb)
        for t in range(26, 30):
            out = e.step([StepEntry(sa, [a[t]], [0])]).cpu()
            rows.append((out[0], ra[t]))
        e.release_slot(sa)
        for got, want in rows:
            assert float((got - want).abs().max()) <= 2e-5 * float(ra.abs().max())


# ------------------------------------------------------------------- toy feed-forward with routing, toy positions
def _register_toy_ffn_and_position():
    """Two more kinds defined here, outside the library: a feed-forward that routes each token to one of its
    ReLU experts by the largest of the token's first features, and a position encoding that the attention
    mixer consumes like rotary frequencies (positions divided by a constant: linear interpolation)."""
    import numpy as np
    from cpi_b200.parts import FeedForward, Position, RotaryEncoding, register_feed_forward, register_position
    from cpi_b200.weights import TensorReq

    @register_feed_forward("toy_routed_relu")
    class RoutedRelu(FeedForward):
        def __init__(self, spec, prefix="", workspace=None):
            super().__init__(spec, prefix)
            self.h, self.i, self.e = int(spec["hidden_size"]), int(spec["inner"]), int(spec["experts"])

        def requirements(self):
            return [TensorReq(self.prefix + "ffn.w1", (self.e, self.i, self.h)),
                    TensorReq(self.prefix + "ffn.w2", (self.e, self.h, self.i))]

        def load(self, source, device):
            self.w1 = source.get(self.prefix + "ffn.w1", device).float()
            self.w2 = source.get(self.prefix + "ffn.w2", device).float()

        def forward(self, h, residual, batch):
            x = h.float()
            which = x[:, :self.e].argmax(-1)                       # the routing: a function of the token alone
            for e in range(self.e):
                rows = (which == e).nonzero().flatten()
                if rows.numel():
                    residual[rows] += torch.relu(x[rows] @ self.w1[e].T) @ self.w2[e].T

    @register_position("toy_interpolated")
    class Interpolated(Position):
        def __init__(self, spec, prefix=""):
            super().__init__(spec, prefix)
            d, div = int(spec["head_dim"]), float(spec["divide_by"])
            self.frequencies = (np.float32(1.0 / div) *
                                np.float32(spec["theta"]) ** (-np.arange(d // 2, dtype=np.float32) * 2 / d)).astype(np.float32)
            self.inv_freq = None

        def prepare(self, device):
            self.inv_freq = torch.from_numpy(self.frequencies).to(device)

        def encoding(self):
            return RotaryEncoding(self.inv_freq, interleaved=True)

    return RoutedRelu, Interpolated


def test_toy_routed_feed_forward_and_toy_positions_register_build_and_step():
    """A model whose feed-forward and position encoding are defined in this test, around the library's
    attention mixer: whole prompts, an unequal batch, and decoding, against plain formulas (in float32: the
    toy routing is an arg-max of raw features, which bfloat16 rounding would flip now and then)."""
    dtype = "float32"
    from cpi_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.engine.model import tensor_requirements
    from cpi_b200.weights import DictSource, RandomSource
    _, Interp = _register_toy_ffn_and_position()
    H, V, NH, NKV, D, I, E = 64, 120, 4, 2, 32, 48, 3
    pos = PartSpec("toy_interpolated", {"head_dim": D, "theta": 5000.0, "divide_by": 4.0})
    norm = lambda w: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "weight": w})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": D,
                                  "softmax_scale": D ** -0.5, "position": pos, "qk_norm": False, "qk_norm_eps": 0.0,
                                  "qk_norm_order": "after_rope", "window": {"kind": "sliding", "size": 7},
                                  "query_temperature": None})
    layers = tuple(LayerSpec(prefix=f"l{i}.", block=PartSpec("pre_norm"), mixer=attn,
                             feed_forward=PartSpec("toy_routed_relu", {"hidden_size": H, "inner": I, "experts": E}),
                             mixer_norm=norm("n1.weight"), feed_forward_norm=norm("n2.weight")) for i in range(2))
    spec = ModelSpec(architecture="Toy2", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"weight": "emb.weight"}), layers=layers,
                     run_order=(RunEntry(0), RunEntry(1)), final_norm=norm("norm.weight"),
                     head=PartSpec("linear_head", {"weight": "head.weight"}), initializer_range=0.2)
    src = RandomSource(tensor_requirements(spec), 5, 0.2)
    drawn = {n: src.get(n, "cpu") for n in src.names()}
    W = {n: t.float() for n, t in drawn.items()}
    e = Engine(spec, DictSource(drawn), dtype=dtype, max_tokens=512)
    assert not e.use_graphs                  # the toy feed-forward synchronises: its steps are not captured
    freqs = Interp(pos).frequencies

    def plain(tokens):
        n = len(tokens)
        p = list(range(n))
        x = W["emb.weight"][tokens]
        for i in range(2):
            h = P.rmsnorm(x, W[f"l{i}.n1.weight"], 1e-5)
            q = (h @ W[f"l{i}.self_attn.q_proj.weight"].T).reshape(n, NH, D)
            k = (h @ W[f"l{i}.self_attn.k_proj.weight"].T).reshape(n, NKV, D)
            v = (h @ W[f"l{i}.self_attn.v_proj.weight"].T).reshape(n, NKV, D)
            q, k = P.rope(q, p, freqs, "interleaved"), P.rope(k, p, freqs, "interleaved")
            pt = torch.tensor(p)
            mask = (pt[None, :] <= pt[:, None]) & (pt[None, :] > pt[:, None] - 7)
            x = x + P.attention(q, k, v, mask, D ** -0.5) @ W[f"l{i}.self_attn.o_proj.weight"].T
            h2 = P.rmsnorm(x, W[f"l{i}.n2.weight"], 1e-5)
            which = h2[:, :E].argmax(-1)
            y = torch.zeros_like(x)
            for ex in range(E):
                rows = (which == ex).nonzero().flatten()
                y[rows] = torch.relu(h2[rows] @ W[f"l{i}.ffn.w1"][ex].T) @ W[f"l{i}.ffn.w2"][ex].T
            x = x + y
        return P.rmsnorm(x, W["norm.weight"], 1e-5) @ W["head.weight"].T

    a, b = tiny.random_tokens(40, V, 1), tiny.random_tokens(13, V, 2)
    ra, rb = plain(a), plain(b)
    tol = 2e-5 * float(ra.abs().max())
    sa, sb = e.acquire_slot(), e.acquire_slot()
    out = e.step([StepEntry(sa, a[:33], [0, 32]), StepEntry(sb, b[:12], [11])]).float().cpu()
    rows = [(out[0], ra[0]), (out[1], ra[32]), (out[2], rb[11])]
    out = e.step([StepEntry(sa, [a[33]], [0]), StepEntry(sb, [b[12]], [0])]).float().cpu()
    rows += [(out[0], ra[33]), (out[1], rb[12])]
    e.release_slot(sb)
    for t in range(34, 40):
        rows.append((e.step([StepEntry(sa, [a[t]], [0])]).float().cpu()[0], ra[t]))
    e.release_slot(sa)
    e.check_device_errors()
    for got, want in rows:
        assert float((got - want).abs().max()) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_that_biases_the_scores_and_one_the_mixer_refuses(dtype):
    """Positions need not rotate anything: a position part defined here describes itself as a bias on the scores
    by (head, distance), with a slope per head and distances beyond the table's end sharing its last column.
    The attention mixer takes it (on its general kernel) in prompts, unequal batches and decoding; a part that
    describes itself as something the mixer's kernels do not know is refused when the model is built."""
    from dataclasses import dataclass
    from cpi_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.engine.model import tensor_requirements
    from cpi_b200.parts import Position, ScoreBias, register_position
    from cpi_b200.weights import DictSource, RandomSource
    H, V, NH, NKV, D, I, N_DIST = 64, 90, 4, 2, 64, 96, 24

    @register_position("toy_distance_bias")
    class DistanceBias(Position):
        graph_safe = True

        def __init__(self, spec, prefix=""):
            super().__init__(spec, prefix)
            slopes = torch.tensor([float(spec["slope"]) * (h + 1) for h in range(int(spec["heads"]))])
            self.table_cpu = -slopes[:, None] * torch.arange(int(spec["distances"]), dtype=torch.float32)[None, :]
            self.table = None

        def prepare(self, device):
            self.table = self.table_cpu.contiguous().to(device)

        def encoding(self):
            return ScoreBias(self.table)

    @dataclass
    class Unknown:
        anything: int = 0

    @register_position("toy_unknown_kind")
    class Strange(Position):
        def encoding(self):
            return Unknown()

    def spec_with(pos):
        norm = lambda w: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "weight": w})
        attn = PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": D,
                                      "softmax_scale": D ** -0.5, "position": pos, "qk_norm": False,
                                      "qk_norm_eps": 0.0, "window": {"kind": "full", "size": 0},
                                      "query_temperature": None})
        ffn = PartSpec("dense_swiglu", {"hidden_size": H, "intermediate_size": I})
        layers = tuple(LayerSpec(prefix=f"l{i}.", block=PartSpec("pre_norm"), mixer=attn, feed_forward=ffn,
                                 mixer_norm=norm("n1.weight"), feed_forward_norm=norm("n2.weight")) for i in range(2))
        return ModelSpec(architecture="ToyBias", hidden_size=H, vocab_size=V,
                         embedding=PartSpec("token_embedding", {"weight": "emb.weight"}), layers=layers,
                         run_order=(RunEntry(0), RunEntry(1)), final_norm=norm("norm.weight"),
                         head=PartSpec("linear_head", {"weight": "head.weight"}), initializer_range=0.2)

    pos = PartSpec("toy_distance_bias", {"heads": NH, "slope": 0.11, "distances": N_DIST})
    spec = spec_with(pos)
    src = RandomSource(tensor_requirements(spec), 9, 0.2)
    drawn = {n: src.get(n, "cpu") for n in src.names()}
    W = {n: t.float() for n, t in drawn.items()}
    with pytest.raises(TypeError, match="toy_unknown_kind.*Unknown"):
        Engine(spec_with(PartSpec("toy_unknown_kind", {})), DictSource(drawn), dtype=dtype, max_tokens=64)
    e = Engine(spec, DictSource(drawn), dtype=dtype, max_tokens=512)
    assert e.use_graphs
    table = DistanceBias(pos).table_cpu

    def plain(tokens):
        n = len(tokens)
        x = W["emb.weight"][tokens]
        pt = torch.arange(n)
        dist = (pt[:, None] - pt[None, :]).clamp(0, N_DIST - 1)
        causal = pt[None, :] <= pt[:, None]
        for i in range(2):
            h = P.rmsnorm(x, W[f"l{i}.n1.weight"], 1e-5)
            q = (h @ W[f"l{i}.self_attn.q_proj.weight"].T).reshape(n, NH, D)
            k = (h @ W[f"l{i}.self_attn.k_proj.weight"].T).reshape(n, NKV, D)
            v = (h @ W[f"l{i}.self_attn.v_proj.weight"].T).reshape(n, NKV, D)
            out = torch.empty(n, NH, D)
            for hd in range(NH):
                s = (q[:, hd] @ k[:, hd // (NH // NKV)].T) * D ** -0.5 + table[hd][dist]
                s = s.masked_fill(~causal, float("-inf"))
                out[:, hd] = torch.softmax(s, -1) @ v[:, hd // (NH // NKV)]
            x = x + out.reshape(n, NH * D) @ W[f"l{i}.self_attn.o_proj.weight"].T
            h2 = P.rmsnorm(x, W[f"l{i}.n2.weight"], 1e-5)
            f = f"l{i}.feed_forward."
            x = x + P.swiglu_mlp(h2, W[f + "gate_proj.weight"], W[f + "up_proj.weight"], W[f + "down_proj.weight"])
        return P.rmsnorm(x, W["norm.weight"], 1e-5) @ W["head.weight"].T

    a, b = tiny.random_tokens(70, V, 1), tiny.random_tokens(13, V, 2)
    ra, rb = plain(a), plain(b)
    tol = (2e-5 if dtype == "float32" else 2e-2) * float(ra.abs().max())
    sa, sb = e.acquire_slot(), e.acquire_slot()
    out = e.step([StepEntry(sa, a[:50], [0, 30, 49]), StepEntry(sb, b[:12], [11])]).float().cpu()
    rows = [(out[0], ra[0]), (out[1], ra[30]), (out[2], ra[49]), (out[3], rb[11])]
    out = e.step([StepEntry(sa, [a[50]], [0]), StepEntry(sb, [b[12]], [0])]).float().cpu()
    rows += [(out[0], ra[50]), (out[1], rb[12])]
    e.release_slot(sb)
    for t in range(51, 70):
        rows.append((e.step([StepEntry(sa, [a[t]], [0])]).float().cpu()[0], ra[t]))
    e.release_slot(sa)
    e.check_device_errors()
    for got, want in rows:
        assert float((got - want).abs().max()) <= tol


def test_toy_mixer_with_one_latent_stream_per_position_registers_builds_and_steps():
    """A mixer that keeps neither keys nor values but ONE compressed vector per position (a stream of its own
    name and width in the paged cache) and attends over those: defined here, registered, built and stepped without
    a change to the library: whole prompts, an unequal batch, prompt tokens on a filled cache, decoding, and a
    second round in the slots and pages that the first gave back."""
    from cpi_b200.cache import KVRequirement
    from cpi_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from cpi_b200.engine import Engine, StepEntry
    from cpi_b200.engine.model import tensor_requirements
    from cpi_b200.parts import Mixer, register_mixer
    from cpi_b200.weights import DictSource, RandomSource, TensorReq
    H, V, I, L, NH = 48, 70, 64, 24, 3

    @register_mixer("toy_latent_attention")
    class LatentAttention(Mixer):
        def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
            super().__init__(spec, prefix)

        def requirements(self):
            return [TensorReq(self.prefix + "lat.down", (L, H)), TensorReq(self.prefix + "lat.q", (NH * L, H)),
                    TensorReq(self.prefix + "lat.out", (H, NH * L))]

        def load(self, source, device):
            self.wd, self.wq, self.wo = (source.get(self.prefix + n, device).float() for n in ("lat.down", "lat.q", "lat.out"))

        def kv_requirement(self):
            return KVRequirement(0, 0, streams=(("latent", 1, L),))

        def forward(self, h, residual, batch, cache):
            pages, table, page = cache.stream("latent")                 # [pages, 1, page, L]
            x = h.float()
            off = 0
            for slot, start, n in zip(batch.slots, batch.starts, batch.n_new):
                pos = torch.arange(start, start + n, device=h.device)
                pg = table[slot, (pos // page).long()].long()
                pages[pg, 0, (pos % page).long()] = (x[off:off + n] @ self.wd.T).to(pages.dtype)
                allp = torch.arange(0, start + n, device=h.device)
                c = pages[table[slot, (allp // page).long()].long(), 0, (allp % page).long()].float()   # [start + n, L]
                q = (x[off:off + n] @ self.wq.T).view(n, NH, L)
                s = torch.einsum("nhl,tl->nht", q, c) * L ** -0.5
                s = s.masked_fill(allp[None, None, :] > pos[:, None, None], float("-inf"))
                o = torch.einsum("nht,tl->nhl", torch.softmax(s, -1), c).reshape(n, NH * L)
                residual[off:off + n] += o @ self.wo.T
                off += n

    norm = lambda w: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "weight": w})
    layers = tuple(LayerSpec(prefix=f"l{i}.", block=PartSpec("pre_norm"), mixer=PartSpec("toy_latent_attention", {}),
                             feed_forward=PartSpec("dense_swiglu", {"hidden_size": H, "intermediate_size": I}),
                             mixer_norm=norm("n1.weight"), feed_forward_norm=norm("n2.weight")) for i in range(2))
    spec = ModelSpec(architecture="ToyLatent", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"weight": "emb.weight"}), layers=layers,
                     run_order=(RunEntry(0), RunEntry(1)), final_norm=norm("norm.weight"),
                     head=PartSpec("linear_head", {"weight": "emb.weight"}), initializer_range=0.15)
    src = RandomSource(tensor_requirements(spec), 6, 0.15)
    drawn = {n: src.get(n, "cpu") for n in src.names()}
    W = {n: t.float() for n, t in drawn.items()}
    e = Engine(spec, DictSource(drawn), dtype="float32", max_tokens=256)
    assert len(e.cache.groups) == 1 and sorted(e.cache.groups[0].streams) == ["latent"]
    assert e.cache.groups[0].streams["latent"].shape == (2, 4, 1, 64, L)

    def plain(tokens):
        n = len(tokens)
        x = W["emb.weight"][tokens]
        causal = torch.arange(n)[None, :] <= torch.arange(n)[:, None]
        for i in range(2):
            h = P.rmsnorm(x, W[f"l{i}.n1.weight"], 1e-5)
            c = h @ W[f"l{i}.lat.down"].T
            q = (h @ W[f"l{i}.lat.q"].T).view(n, NH, L)
            s = torch.einsum("nhl,tl->nht", q, c) * L ** -0.5
            s = s.masked_fill(~causal[:, None, :], float("-inf"))
            x = x + torch.einsum("nht,tl->nhl", torch.softmax(s, -1), c).reshape(n, NH * L) @ W[f"l{i}.lat.out"].T
            h2 = P.rmsnorm(x, W[f"l{i}.n2.weight"], 1e-5)
            f = f"l{i}.feed_forward."
            x = x + P.swiglu_mlp(h2, W[f + "gate_proj.weight"], W[f + "up_proj.weight"], W[f + "down_proj.weight"])
        return P.rmsnorm(x, W["norm.weight"], 1e-5) @ W["emb.weight"].T

    a, b = tiny.random_tokens(100, V, 1), tiny.random_tokens(12, V, 2)
    ra, rb = plain(a), plain(b)
    tol = 2e-5 * float(ra.abs().max())
    for round_ in range(2):
        sa, sb = e.acquire_slot(), e.acquire_slot()
        out = e.step([StepEntry(sa, a[:60], [0, 59]), StepEntry(sb, b[:9], [8])]).cpu()
        rows = [(out[0], ra[0]), (out[1], ra[59]), (out[2], rb[8])]
        out = e.step([StepEntry(sa, a[60:90], [0, 29]), StepEntry(sb, [b[9]], [0])]).cpu()     # across a page boundary
        rows += [(out[0], ra[60]), (out[1], ra[89]), (out[2], rb[9])]
        e.release_slot(sb)
        for t in range(90, 100):
            rows.append((e.step([StepEntry(sa, [a[t]], [0])]).cpu()[0], ra[t]))
        e.release_slot(sa)
        e.cache.check_consistency()
        for got, want in rows:
            assert float((got - want).abs().max()) <= tol
