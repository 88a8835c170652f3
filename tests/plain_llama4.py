"""Plain, slow float32 implementation of the Llama4 text decoder: the tests' oracle.

Whole sequences, no cache, one function per part, on the CPU.  It shares no code
with `cpi_b200`: it reads config.json as a dictionary and the tensors by their
names, and is written from the reference's formulas.  Citations are
file:line of kurulav1/cpi; "REF" abbreviates src/engine/llama4_cpu_engine.cpp.

What the reference's forward computes (REF:293-333) is one layer kind: RMSNorm,
q/k/v projections, weightless per-head RMS norm of q and k, half-split RoPE with
llama3 frequency scaling, causal attention, output projection, RMSNorm, top-1
routed expert without a gate value plus a shared expert.  `tests/golden/`
compares this file with the compiled reference engine on that subset.  The
options the reference does not have (layers without position encoding, chunked
attention, query temperature, sigmoid gates, top-k > 1, dense layers, tied
head, norm after RoPE) rest on the formulas written in each function below.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


# --------------------------------------------------------------------------- config
def read_config(model_dir: str) -> dict:
    """Flat dictionary of the text decoder's keys with the same defaults the library documents."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    arch = raw["architectures"][0]
    c = dict(raw.get("text_config", raw))
    for k in ("tie_word_embeddings",):
        if k not in c and k in raw:
            c[k] = raw[k]
    c["_prefix"] = "language_model." if arch == "Llama4ForConditionalGeneration" else ""
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("intermediate_size_mlp", c["intermediate_size"])
    c.setdefault("num_experts_per_tok", 1)
    c.setdefault("interleave_moe_layer_step", 1)
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 500000.0)
    c.setdefault("rope_scaling", None)
    c.setdefault("nope_layer_interval", 4)
    if c.get("attention_chunk_size", 8192) is None:
        c["attention_chunk_size"] = 0
    c.setdefault("attention_chunk_size", 8192)
    c.setdefault("use_qk_norm", True)
    c.setdefault("attn_temperature_tuning", True)
    c.setdefault("floor_scale", 8192)
    c.setdefault("attn_scale", 0.1)
    c.setdefault("tie_word_embeddings", False)
    c.setdefault("rope_pairing", "half_split")
    c.setdefault("qk_norm_order", "after_rope")
    c.setdefault("qk_norm_scope", "rope_layers")
    c.setdefault("router_gate", "sigmoid_input")
    return c


def read_weights(model_dir: str) -> dict:
    """All tensors as float32 (bf16 widens exactly, as REF:24-29 does with a 16-bit shift)."""
    from safetensors.torch import load_file
    out = {}
    for f in sorted(os.listdir(model_dir)):
        if f.endswith(".safetensors"):
            for k, v in load_file(os.path.join(model_dir, f)).items():
                out.setdefault(k, v.to(torch.float32))
    return out


def layer_is_moe(c: dict, i: int) -> bool:
    if c.get("moe_layers") is not None:
        return i in c["moe_layers"]
    return (i + 1) % c["interleave_moe_layer_step"] == 0


def layer_uses_rope(c: dict, i: int) -> bool:
    if c.get("no_rope_layers"):
        return bool(c["no_rope_layers"][i])
    if c.get("layer_types"):
        return c["layer_types"][i] == "chunked_attention"
    n = c["nope_layer_interval"]
    return True if n <= 0 else (i + 1) % n != 0


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x = Emb[token]  (REF:294-298)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)].clone()


def rmsnorm(x: torch.Tensor, w, eps: float) -> torch.Tensor:
    """out = x * 1/sqrt(mean(x^2) + eps) * w over the last axis; w may be None (REF:47-62)."""
    inv = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    y = x * inv
    return y if w is None else y * w


def rope_frequencies(c: dict) -> np.ndarray:
    """theta_d for d < D/2 in float32, with llama3 scaling when configured (REF:446-464).

    wavelen = 2*pi/theta_d; wavelen > orig/low: theta_d /= factor; wavelen >= orig/high:
    smooth = (orig/wavelen - low)/(high - low), theta_d = (1-smooth)*theta_d/factor + smooth*theta_d.
    """
    D = c["head_dim"]
    half = D // 2
    f32 = np.float32
    out = np.zeros(half, dtype=np.float32)
    rs = c["rope_scaling"]
    for d in range(half):
        theta_d = f32(np.power(f32(c["rope_theta"]), f32(-2.0) * f32(d) / f32(D), dtype=np.float32))
        if rs is not None:
            orig = f32(rs["original_max_position_embeddings"])
            low, high, factor = f32(rs["low_freq_factor"]), f32(rs["high_freq_factor"]), f32(rs["factor"])
            wavelen = f32(2.0) * f32(3.14159265358979323846) / theta_d
            if wavelen > orig / low:
                theta_d = theta_d / factor
            elif wavelen >= orig / high:
                smooth = (orig / wavelen - low) / (high - low)
                theta_d = (f32(1.0) - smooth) * (theta_d / factor) + smooth * theta_d
        out[d] = theta_d
    return out


def rope(x: torch.Tensor, positions, freqs: np.ndarray, pairing: str) -> torch.Tensor:
    """Rotate x [n, heads, D] at absolute positions (REF:167-193; angle = float(p)*theta_d, REF:467).

    half_split pairs (d, d + D/2) as the reference does; interleaved pairs (2d, 2d+1).
    x'[a] = x[a]*cos - x[b]*sin ; x'[b] = x[a]*sin + x[b]*cos.
    """
    n, _, D = x.shape
    half = D // 2
    ang = np.asarray(positions, dtype=np.float32)[:, None] * freqs[None, :]       # float32 product
    cos = torch.from_numpy(np.cos(ang).astype(np.float32))[:, None, :]
    sin = torch.from_numpy(np.sin(ang).astype(np.float32))[:, None, :]
    out = torch.empty_like(x)
    if pairing == "half_split":
        a, b = x[..., :half], x[..., half:]
        out[..., :half] = a * cos - b * sin
        out[..., half:] = a * sin + b * cos
    else:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    return out


def query_temperature(q: torch.Tensor, positions, floor_scale: float, attn_scale: float) -> torch.Tensor:
    """q *= 1 + attn_scale * ln(floor((p+1)/floor_scale) + 1), on layers without position encoding.

    The reference has no such step; this is the formula of the library's documentation.
    """
    p = torch.as_tensor(positions, dtype=torch.float32)
    s = 1.0 + attn_scale * torch.log(torch.floor((p + 1.0) / floor_scale) + 1.0)
    return q * s[:, None, None]


def attention_scores_mask(n: int, positions, chunk: int) -> torch.Tensor:
    """mask[i, j] True where query i may see key j: causal (REF:208), same chunk of `chunk` positions if > 0."""
    p = torch.as_tensor(positions, dtype=torch.long)
    ok = p[None, :] <= p[:, None]
    if chunk > 0:
        ok &= (p[None, :] // chunk) == (p[:, None] // chunk)
    return ok


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, scale: float) -> torch.Tensor:
    """Softmax attention with grouped heads (REF:195-250).

    s = (q_h . k_{h // G}) * scale; m = max; e = exp(s - m); P = e / max(sum e, 1e-20); out = sum P v.
    q [n, NH, D], k/v [n, NKV, D] -> [n, NH*D].
    """
    n, NH, D = q.shape
    G = NH // k.shape[1]
    out = torch.empty(n, NH, D)
    for h in range(NH):
        kh, vh = k[:, h // G, :], v[:, h // G, :]
        s = (q[:, h, :] @ kh.T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        P = e / torch.clamp(e.sum(-1, keepdim=True), min=1e-20)
        out[:, h, :] = P @ vh
    return out.reshape(n, NH * D)


def attention_part(c: dict, W: dict, pre: str, i: int, h: torch.Tensor, positions) -> torch.Tensor:
    """The whole mixer of layer i on normed input h [n, H] -> [n, H] (REF:304-323)."""
    NH, NKV, D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    n = h.shape[0]
    q = (h @ W[pre + "self_attn.q_proj.weight"].T).reshape(n, NH, D)
    k = (h @ W[pre + "self_attn.k_proj.weight"].T).reshape(n, NKV, D)
    v = (h @ W[pre + "self_attn.v_proj.weight"].T).reshape(n, NKV, D)
    uses_rope = layer_uses_rope(c, i)
    has_norm = c["use_qk_norm"] and (c["qk_norm_scope"] == "all_layers" or uses_rope)
    eps = c["rms_norm_eps"]

    def qk_norm(q, k):
        # weightless per-head RMS norm (REF:308-317; weights only if the tensors exist, REF:440-443)
        return (rmsnorm(q, W.get(pre + "self_attn.q_norm.weight"), eps),
                rmsnorm(k, W.get(pre + "self_attn.k_norm.weight"), eps))

    if has_norm and c["qk_norm_order"] == "before_rope":
        q, k = qk_norm(q, k)
    if uses_rope:
        fr = rope_frequencies(c)
        q = rope(q, positions, fr, c["rope_pairing"])
        k = rope(k, positions, fr, c["rope_pairing"])
    if has_norm and c["qk_norm_order"] == "after_rope":
        q, k = qk_norm(q, k)
    if (not uses_rope) and c["attn_temperature_tuning"]:
        q = query_temperature(q, positions, float(c["floor_scale"]), float(c["attn_scale"]))
    chunk = c["attention_chunk_size"] if uses_rope else 0
    mask = attention_scores_mask(n, positions, chunk)
    a = attention(q, k, v, mask, 1.0 / math.sqrt(D))          # scale 1/sqrt(D): REF:197
    return a @ W[pre + "self_attn.o_proj.weight"].T


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x))  (REF:64-66)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate h) * (up h)), weights [out, in] (shared expert: REF:279-287)."""
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def router_top_k(h: torch.Tensor, w_router: torch.Tensor, k: int):
    """Router logits [n, E] and the k best experts per token, ties to the lowest index.

    The reference takes the single best with a strict '>' scanning upward (REF:256-263).
    """
    logits = h @ w_router.T
    n, E = logits.shape
    idx = torch.empty(n, k, dtype=torch.long)
    for t in range(n):
        row = logits[t].tolist()
        taken = []
        for _ in range(k):
            best = -1
            for e in range(E):
                if e in taken:
                    continue
                if best < 0 or row[e] > row[best]:
                    best = e
            taken.append(best)
        idx[t] = torch.tensor(taken)
    return logits, idx


def routed_experts(h: torch.Tensor, w_router, w_gate_up, w_down, k: int, gate_mode: str, forced_idx=None):
    """Sum over the token's k experts (REF:265-277 for k = 1 without gate).

    gate g = sigmoid(router logit).  sigmoid_input: the expert sees g*h; sigmoid_output: its
    output is scaled by g; none: no gate (the reference).  gate_up [E, H, 2I] is applied as
    h @ W; its first I columns are the gate, the rest the up projection.  down [E, I, H].
    """
    logits, idx = router_top_k(h, w_router, k)
    if forced_idx is not None:          # tests: follow another implementation's choice at near-ties
        idx = torch.as_tensor(forced_idx, dtype=torch.long).reshape(idx.shape)
    n = h.shape[0]
    I = w_down.shape[1]
    out = torch.zeros(n, w_down.shape[2])
    for t in range(n):
        for j in range(k):
            e = int(idx[t, j])
            g = 1.0 / (1.0 + torch.exp(-logits[t, e]))
            u = h[t] * g if gate_mode == "sigmoid_input" else h[t]
            gu = u @ w_gate_up[e]
            a = silu(gu[:I]) * gu[I:]
            y = a @ w_down[e]
            if gate_mode == "sigmoid_output":
                y = y * g
            out[t] += y
    return out, logits, idx


def feed_forward_part(c: dict, W: dict, pre: str, i: int, h: torch.Tensor, forced_idx=None):
    """Layer i's feed-forward on normed input h: routed + shared experts (REF:252-291) or a dense SwiGLU."""
    if layer_is_moe(c, i):
        f = pre + "feed_forward."
        routed, logits, idx = routed_experts(h, W[f + "router.weight"], W[f + "experts.gate_up_proj"],
                                             W[f + "experts.down_proj"], c["num_experts_per_tok"],
                                             c["router_gate"], forced_idx)
        shared = swiglu_mlp(h, W[f + "shared_expert.gate_proj.weight"], W[f + "shared_expert.up_proj.weight"],
                            W[f + "shared_expert.down_proj.weight"])
        return routed + shared, (logits, idx)
    f = pre + "feed_forward."
    return swiglu_mlp(h, W[f + "gate_proj.weight"], W[f + "up_proj.weight"], W[f + "down_proj.weight"]), None


# --------------------------------------------------------------------------- whole model
def forward(c: dict, W: dict, tokens, return_router: bool = False, forced_routing=None):
    """Logits [n, V] at every position of one sequence (REF:293-333 for every token at once).

    forced_routing: optional {layer: expert indices [n, k]} that replace the router's own choice; the
    router logits are still returned, so a test can check that a forced choice was a near-tie.
    """
    p = c["_prefix"]
    n = len(tokens)
    positions = list(range(n))
    x = embedding(W[p + "model.embed_tokens.weight"], tokens)
    eps = c["rms_norm_eps"]
    routing = []
    for i in range(c["num_hidden_layers"]):
        pre = f"{p}model.layers.{i}."
        h = rmsnorm(x, W[pre + "input_layernorm.weight"], eps)
        x = x + attention_part(c, W, pre, i, h, positions)
        h2 = rmsnorm(x, W[pre + "post_attention_layernorm.weight"], eps)
        y, r = feed_forward_part(c, W, pre, i, h2, None if forced_routing is None else forced_routing.get(i))
        routing.append(r)
        x = x + y
    xn = rmsnorm(x, W[p + "model.norm.weight"], eps)
    head = W[p + "model.embed_tokens.weight"] if c["tie_word_embeddings"] else W[p + "lm_head.weight"]
    logits = xn @ head.T
    return (logits, routing) if return_router else logits


def min_router_margin(routing, k: int) -> float:
    """Smallest gap between the k-th and (k+1)-th router logit over all tokens and MoE layers."""
    m = float("inf")
    for r in routing:
        if r is None:
            continue
        logits, _ = r
        if logits.shape[1] <= k:
            continue
        s = torch.sort(logits, dim=-1, descending=True).values
        m = min(m, float((s[:, k - 1] - s[:, k]).min()))
    return m


def greedy_generate(c: dict, W: dict, prompt, max_new: int, stop_ids=()):
    """Greedy continuation by re-running the whole sequence each step (first maximum wins)."""
    seq = list(prompt)
    out = []
    for _ in range(max_new):
        logits = forward(c, W, seq)[-1]
        nxt = int(torch.argmax(logits))
        out.append(nxt)
        seq.append(nxt)
        if nxt in stop_ids:
            break
    return out
