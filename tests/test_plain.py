"""The plain implementation: against the reference's own CPU engine, and its parts against each other."""
import hashlib
import os

import numpy as np
import pytest
import torch

import plain_llama4 as P
import tiny

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
_golden_skipped = set()


@pytest.mark.parametrize("name,file", [("R", "tiny_r_reference.npz"), ("R2", "tiny_r2_reference.npz")])
def test_plain_matches_reference_cpu_engine(name, file):
    """Logits of kurulav1/cpi's unmodified llama4_cpu_engine.cpp (made by tests/golden/make_golden.py) at two
    points that differ in every size the reference's engine lets one choose."""
    g = np.load(os.path.join(GOLDEN, file))
    d = tiny.make_model_dir(name)
    with open(os.path.join(d, "model.safetensors"), "rb") as f:
        if hashlib.sha256(f.read()).hexdigest() != str(g["digest"]):
            _golden_skipped.add(name)
            pytest.skip("the random weights drawn here differ from those the golden file was made with: "
                        "run tests/golden/make_golden.py again")
    c, W = P.read_config(d), P.read_weights(d)
    logits = P.forward(c, W, g["tokens"].tolist()).numpy()
    err = np.abs(logits - g["logits"]).max()
    assert err <= 5e-6 * np.abs(g["logits"]).max(), err
    assert (logits.argmax(-1) == g["logits"].argmax(-1)).all()


def test_a_golden_point_was_compared():
    """One stale golden file is a skip; with both stale the plain implementation would rest on nothing."""
    assert len(_golden_skipped) < 2, ("both golden files were made with other random weights than those drawn "
                                      "here: run tests/golden/make_golden.py again")


def test_rmsnorm_and_silu():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0 / 12.5 ** 0.5 * 2, 4.0 / 12.5 ** 0.5 * 0.5]]))
    assert torch.allclose(P.silu(torch.tensor([0.0, 1.0])), torch.tensor([0.0, 1.0 / (1 + np.exp(-1.0))]).float())


def test_rope_frequencies_llama3_bands():
    c = {"head_dim": 16, "rope_theta": 500000.0,
         "rope_scaling": {"factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                          "original_max_position_embeddings": 64}}
    f = P.rope_frequencies(c)
    base = np.array([500000.0 ** (-2.0 * d / 16) for d in range(8)])
    assert np.isclose(f[0], 1.0)                              # short wavelength: unchanged
    assert np.isclose(f[-1], base[-1] / 16.0, rtol=1e-5)      # long wavelength: divided by the factor
    assert all(f[i] <= base[i] * (1 + 1e-6) for i in range(8))
    c["rope_scaling"] = None
    assert np.allclose(P.rope_frequencies(c), base, rtol=1e-6)


def test_rope_pairings_are_permutations_of_each_other():
    torch.manual_seed(0)
    x = torch.randn(5, 2, 8)
    fr = np.array([1.0, 0.5, 0.25, 0.125], dtype=np.float32)
    pos = [0, 3, 7, 8, 100]
    hs = P.rope(x, pos, fr, "half_split")
    perm = [0, 4, 1, 5, 2, 6, 3, 7]                           # interleaved index -> half-split index
    il = P.rope(x[..., perm], pos, fr, "interleaved")
    assert torch.allclose(il, hs[..., perm], atol=1e-6)
    assert torch.allclose(hs[0], x[0])                        # position 0 is the identity
    assert torch.allclose(hs.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_mask_chunks_and_causality():
    m = P.attention_scores_mask(6, range(6), 4)
    assert m[3].tolist() == [True, True, True, True, False, False]
    assert m[4].tolist() == [False, False, False, False, True, False]
    assert P.attention_scores_mask(3, range(3), 0)[2].tolist() == [True, True, True]


def test_attention_far_key_dominates():
    """One key scaled up must take all the weight: out = its value."""
    torch.manual_seed(1)
    n, D = 40, 8
    q, k, v = torch.randn(n, 2, D), torch.randn(n, 1, D), torch.randn(n, 1, D)
    k[3, 0] = q[n - 1, 0] * 50.0
    out = P.attention(q, k, v, P.attention_scores_mask(n, range(n), 0), 1.0).reshape(n, 2, D)
    assert torch.allclose(out[n - 1, 0], v[3, 0], atol=1e-4)


def test_router_ties_go_to_lowest_index_and_top_k():
    h = torch.eye(2)
    w = torch.tensor([[1.0, 0.0], [1.0, 5.0], [1.0, 5.0], [0.0, 0.0]])
    logits, idx = P.router_top_k(h, w, 2)
    assert idx[0].tolist() == [0, 1]          # three-way tie at 1.0: experts 0 and 1
    assert idx[1].tolist() == [1, 2]          # tie at 5.0: lowest index first


def test_temperature_floor():
    q = torch.ones(4, 1, 2)
    out = P.query_temperature(q, [0, 30, 31, 63], 32.0, 0.1)
    assert torch.allclose(out[:2], torch.ones(2, 1, 2))
    assert torch.allclose(out[2], torch.full((1, 2), 1 + 0.1 * np.log(2.0)))
    assert torch.allclose(out[3], torch.full((1, 2), 1 + 0.1 * np.log(3.0)))


@pytest.mark.parametrize("name", ["A", "B"])
def test_prefix_invariance(name):
    """Causality: logits of a prefix do not change when tokens are appended."""
    d = tiny.make_model_dir(name)
    c, W = P.read_config(d), P.read_weights(d)
    t = tiny.random_tokens(45, c["vocab_size"], 3)
    full, part = P.forward(c, W, t), P.forward(c, W, t[:20])
    assert torch.allclose(full[:20], part, atol=1e-6)


def test_layer_kinds_of_config_b():
    d = tiny.make_model_dir("B")
    c = P.read_config(d)
    assert [P.layer_is_moe(c, i) for i in range(6)] == [False, True, False, True, False, True]
    assert [P.layer_uses_rope(c, i) for i in range(6)] == [True, True, False, True, True, False]
    assert c["_prefix"] == "language_model."
