"""Sizes drawn from a seed, beyond the hand-picked ones of the other files: whole configurations of the architecture
through the engine against the plain implementation, products of drawn shapes against float32, and the tensor-core
attention kernels against the general kernel (which `test_gpu_kernels.py` ties to its plain reference)."""
import math
import random
import shutil

import pytest
import torch

import test_gpu_kernels as TK
import tiny
from helpers import Replay, compare_with_plain, run_batched

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from cpi_b200.csrc import lib
    return lib


def drawn_config(rng):
    """A Llama4 configuration with every size and option drawn; half of them with head sizes and widths that the
    bfloat16 path's tensor-core kernels take."""
    tc_like = rng.random() < 0.5
    D = rng.choice([64, 128]) if tc_like else rng.choice([16, 32, 48, 80, 96, 112, 144, 192, 256])
    NKV = rng.choice([1, 2, 3, 5])
    G = rng.choice([1, 2, 3, 5, 8]) if D <= 128 else rng.choice([1, 2])
    mult = 8 if tc_like else rng.choice([2, 4, 6])
    E = rng.randint(1, 9)
    return {
        "architectures": ["Llama4ForCausalLM"],
        "num_hidden_layers": rng.randint(1, 4), "hidden_size": mult * rng.randint(3, 30),
        "num_attention_heads": NKV * G, "num_key_value_heads": NKV, "head_dim": D,
        "intermediate_size": mult * rng.randint(2, 40), "intermediate_size_mlp": mult * rng.randint(2, 40),
        "num_local_experts": E, "num_experts_per_tok": rng.randint(1, min(3, E)),
        "interleave_moe_layer_step": rng.choice([1, 2]),
        "vocab_size": rng.randint(50, 1500), "rms_norm_eps": rng.choice([1e-5, 1e-6, 1e-4]),
        "rope_theta": rng.choice([1e4, 5e5]),
        "rope_scaling": rng.choice([None, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                           "high_freq_factor": 4.0, "original_max_position_embeddings": 64}]),
        "nope_layer_interval": rng.choice([0, 2, 3]), "attention_chunk_size": rng.choice([0, 16, 24, 100, 130]),
        "use_qk_norm": rng.random() < 0.5, "attn_temperature_tuning": rng.random() < 0.5,
        "floor_scale": rng.choice([16, 100]), "attn_scale": 0.1,
        "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 4096,
        "initializer_range": rng.choice([0.02, 0.05]),
        "rope_pairing": rng.choice(["half_split", "interleaved"]),
        "router_gate": rng.choice(["sigmoid_input", "sigmoid_output", "none"]),
        "qk_norm_order": rng.choice(["before_rope", "after_rope"]),
    }


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations_against_plain(seed):
    """Two batches of one to three requests (prompts of 1 to 600 tokens, up to five decoded tokens each, the second
    batch in the slots of the first), steps whole or in pieces of 50 or 129 tokens, in both precisions."""
    from cpi_b200.engine import Engine
    rng = random.Random(4000 + seed)
    cfg = drawn_config(rng)
    d = tiny.make_model_dir(cfg, seed=seed)
    try:
        for dtype in ("float32", "bfloat16"):
            lens = [rng.randint(1, 600) for _ in range(rng.randint(1, 3))]
            reqs = {f"q{i}": (tiny.random_tokens(n + rng.randint(0, 5), cfg["vocab_size"], 31 * seed + i), n)
                    for i, n in enumerate(lens)}
            need = sum(-(-len(t) // 64) * 64 for t, _ in reqs.values())
            cap = rng.choice([None, 50, 129])
            e = Engine.from_model_dir(d, dtype=dtype, max_tokens=need, max_seqs=4,
                                      **({"max_step_tokens": cap} if cap else {}))
            rp = Replay(e)
            pos = run_batched(rp, [reqs, reqs])
            e.check_device_errors()
            worst = compare_with_plain(d, {r: t for r, (t, p) in reqs.items()}, rp, dtype, pos)
            print(f"drawn configuration {seed} {dtype}: hidden {cfg['hidden_size']}, heads "
                  f"{cfg['num_attention_heads']}/{cfg['num_key_value_heads']} x {cfg['head_dim']}, experts "
                  f"{cfg['num_local_experts']} top {cfg['num_experts_per_tok']}, prompts {lens}, pieces {cap}: "
                  f"worst relative error {worst:.2e}")
    finally:
        shutil.rmtree(d, ignore_errors=True)


@pytest.mark.parametrize("seed", range(60))
def test_drawn_products_against_float32(seed):
    """`gemm_tc` (few tokens, any feature count) and `gemm_tc_pair` (512 tokens or more, features in 256s): drawn
    token counts, widths, modes, groups of drawn sizes (empty ones among them), row scales and scattered output
    rows."""
    rng = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    mode = rng.choice([K().MODE_STORE, K().MODE_ADD, K().MODE_SWIGLU])
    G = rng.choice([0, 0, 1, 3, 7, 16])
    pair = rng.random() < 0.4
    if pair:
        N, Kd = 256 * rng.randint(1, 6), 8 * rng.randint(1, 200)
        T = rng.randint(max(512, 64 * G), 3000)
    else:
        N = rng.choice([8, 16, 24, 40, 128, 136, 200, 256, 384, 1000, 1024, 2048 + 64])
        Kd = 8 * rng.randint(1, 300)
        T = rng.choice([1, 2, 3, 5, 8, 9, 16, 17, 31, 33, 64, 65, 100, 128, 129, 200, 257, 300, 511, 700])
    rows = 2 * N if mode == K().MODE_SWIGLU else N
    w = (torch.randn((G, rows, Kd) if G else (rows, Kd), generator=g) * Kd ** -0.5).bfloat16().to(DEV)
    a = torch.randn(T, Kd, generator=g).bfloat16().to(DEV)
    odt = torch.float32 if mode == K().MODE_ADD else (
        torch.bfloat16 if mode == K().MODE_SWIGLU else rng.choice([torch.float32, torch.bfloat16]))
    kw = {}
    if G:
        cuts = sorted(rng.randint(0, T) for _ in range(G - 1))
        counts = [hi - lo for lo, hi in zip([0] + cuts, cuts + [T])]
        offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
        grp = torch.repeat_interleave(torch.arange(G), torch.tensor(counts)).to(DEV)
        kw = dict(m_rows=T, group_offsets=offs, n_groups=G)
        acc = torch.einsum("mk,mnk->mn", a.float(), w.float()[grp])
    else:
        acc = a.float() @ w.float().T
    if rng.random() < 0.5:
        kw["row_scale"] = torch.rand(T, generator=g).to(DEV) + 0.5
        acc = acc * kw["row_scale"][:, None]
    if mode == K().MODE_ADD:
        extra = rng.randint(0, 9)
        out = torch.randn(T + extra, N, generator=g).to(DEV)
        ref = out.clone()
        if rng.random() < 0.5:
            kw["out_rows"] = torch.randperm(T + extra, generator=g)[:T].to(torch.int32).to(DEV)
            ref[kw["out_rows"].long()] += acc
        else:
            ref[:T] += acc
    elif mode == K().MODE_SWIGLU:
        out = torch.zeros(T, N, dtype=odt, device=DEV)
        ref = acc[:, :N] / (1 + torch.exp(-acc[:, :N])) * acc[:, N:]
    else:
        out, ref = torch.zeros(T, N, dtype=odt, device=DEV), acc
    assert (K().gemm_tc_pair if pair else K().gemm_tc)(a, w, out, mode, **kw), (pair, mode, T, N, Kd, G)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0
    tol = (1e-2 if odt == torch.bfloat16 else 3e-5) * max(1.0, float(ref.abs().max()))
    assert float((out.float() - ref).abs().max()) <= tol, (pair, mode, T, N, Kd, G, odt)


@pytest.mark.parametrize("seed", range(40))
def test_drawn_attention_cases_against_the_general_kernel(seed):
    """Prefill: drawn heads and groups, windows of drawn kinds and sizes (1 to 513), sequences that start at drawn
    cache positions, query tiles of drawn sizes.  Decode: drawn lengths and split counts."""
    rng = random.Random(seed)
    D, NKV, G = rng.choice([64, 128]), rng.choice([1, 2, 3, 8]), rng.choice([1, 2, 5, 7, 16])
    NH = NKV * G
    wk = rng.choice(["full", "chunk", "sliding"])
    wsz = 0 if wk == "full" else rng.choice([1, 5, 63, 64, 65, 100, 128, 129, 200, 256, 300, 513])
    seqs = [(rng.choice([0, 0, 1, 63, 64, 70, 128, 200, 300, 511]),
             rng.choice([1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 500])) for _ in range(rng.randint(1, 5))]
    c = TK._prefill_case(NH, NKV, D, (wk, wsz), seqs, seed=seed, tile=rng.choice([256, 256, 128, 200, 17, 1, 255]))
    kw = dict(n_heads=NH, n_kv_heads=NKV, head_dim=D, window_kind=K().WINDOW_KINDS[wk], window_size=wsz,
              scale=rng.choice([1.0 / math.sqrt(D), 0.3]))
    args = (c["k"], c["v"], c["table"], 64, c["token_seq"], c["token_pos"], c["seq_slot"])
    out, gen = torch.full_like(c["q"], float("nan")), torch.empty_like(c["q"])
    K().attention_prefill(c["q"], out, *args, c["tile_tok0"], c["tile_rows"], **kw)
    K().attention_general(c["q"], gen, *args, **kw)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0 and bool(torch.isfinite(out.float()).all())
    assert float((out.float() - gen.float()).abs().max()) <= 2e-2 * max(1.0, float(gen.float().abs().max()))

    lengths = [rng.choice([1, 2, 63, 64, 65, 128, 129, 500, 700, 1500]) for _ in range(rng.randint(1, 6))]
    k, v, table = TK.paged_cache(len(lengths), lengths, NKV, D, 64, torch.bfloat16, seed=seed)
    T = len(lengths)
    q = TK.rnd(T, NH * D, dtype=torch.bfloat16, seed=seed + 9)
    tseq = torch.arange(T, dtype=torch.int32, device=DEV)
    tpos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    slot = torch.arange(1, T + 1, dtype=torch.int32, device=DEV)
    o1, o2 = torch.full_like(q, float("nan")), torch.empty_like(q)
    K().attention_decode(q, o1, k, v, table, 64, tseq, tpos, slot, n_splits=rng.choice([1, 2, 3, 4, 7, 8, 16, 33]), **kw)
    K().attention_general(q, o2, k, v, table, 64, tseq, tpos, slot, **kw)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(o1.float()).all())
    assert float((o1.float() - o2.float()).abs().max()) <= 2e-2 * max(1.0, float(o2.float().abs().max()))
