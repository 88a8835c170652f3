"""Decode and prefill throughput of the Llama4 Scout-sized model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch 8] [--context 4096]
    python bench.py --workload maverick4 | long131k      (two further workloads, a JSON line of their own)

    python bench.py --workload cpu_baseline [--reference-root DIR]      (no GPU needed)

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  `value` is decoded tokens per
second, timed on the device with CUDA events around exactly K engine steps (host token ids in, arg-max
on the device); `e2e` is the same through the Python entry point (`Model.generate`), with every
step's token ids copied from pinned host memory and the sampled ids read back; `points` and `points_e2e`
give both at batch 1 and 64.  Between timed iterations nothing is flushed: one decode step reads tens of
GB of weights, far more than the L2 holds.  `roofline` divides the bytes the timed steps had to read by
their time: every weight a step uses once -- with the experts that THOSE steps touched, counted by running
the same prompts and token feed once more, untimed, with the routing recorded -- and the cache of the live
requests.  `prefill` is one prompt of 2,048 tokens, `prefill_b8` eight of them in one call; `frac` divides
the step's flops by its time and the burst bf16 peak (`frac_of_sustained`: by the rate the library product holds
in a seconds-long loop under the power cap, which is what a step of tens of milliseconds runs at; the clocks
sampled here say the same: ~1.5 of 1.97 GHz), `frac_per_kernel` divides the time the step would
take with every kernel at its own bound (contractions at the tensor peak, but the routed experts at the
larger of that and the time to read their weights once per piece) by the measured time.
For N > 1 GPUs it prints one line that says the library is single-GPU and exits with 2.
`phases` holds device milliseconds per phase of one prefill of 2,048 tokens and of one decode step, taken
after everything else with the steps run eagerly on one stream (so their sum exceeds the step times above).

`--workload contexts`: 12 Scout layers, decode at (batch, context) of (1, 32768), (8, 32768), (64, 8192), (1, 131072)
and (8, 131072), and one prefill of 32,768 tokens, each with its roofline fraction.
`--workload cpu_baseline` times, on the host's cores, the reference's own unmodified CPU engine (compiled from
DIR with tests/golden/ref_harness.cpp, token by token as its generate loop runs it,
src/engine/llama4_cpu_engine.cpp:516-566) and this repository's plain implementation at the two tiny
configurations that lie inside what that engine computes.
`--workload maverick4`: 4 layers with Llama4 Maverick's sizes (dense and 128-expert layers alternate), 32
prompts of 64 to 2,048 tokens, 128 new tokens each.  `--workload long131k`: 12 Scout layers, one prompt of
131,072 tokens (prefilled in pieces), 256 new tokens.  Both run through `Model.generate` and are timed with
its wall-clock phases, second of two runs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of Llama4 Scout (24 of its 48 layers fit one B200 in bfloat16 beside the cache).
SCOUT = {
    "architectures": ["Llama4ForCausalLM"],
    "num_hidden_layers": 24, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 8192, "intermediate_size_mlp": 16384,
    "num_local_experts": 16, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
    "vocab_size": 202048, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "nope_layer_interval": 4, "attention_chunk_size": 8192, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 8192, "attn_scale": 0.1,
    "tie_word_embeddings": False, "max_position_embeddings": 131072, "initializer_range": 0.02,
}
FULL_LAYERS = 48
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)) or None, "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(float(s[0])))
                mx = int(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def layer_weight_bytes(c, touched_experts: float) -> float:
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, E = c["intermediate_size"], c["num_local_experts"]
    attn = (Q + 2 * KV) * H + H * Q
    shared = 3 * I * H
    expert = 3 * I * H
    router = E * H
    return 2.0 * (attn + shared + router + touched_experts * expert + 2 * H)


def decode_step_bytes(c, layers, batch, context, touched_experts) -> float:
    """Bytes one decode step has to read: every weight it uses once and the cache of the live requests (a layer
    with chunked attention reads the keys of the newest position's chunk only)."""
    H, V = c["hidden_size"], c["vocab_size"]
    kv_per_token = 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    C, every = c["attention_chunk_size"], c["nope_layer_interval"]
    keys = 0.0
    for i in range(layers):
        nope = every > 0 and (i + 1) % every == 0
        keys += context if (nope or C <= 0) else (context - 1) % C + 1
    return (layers * layer_weight_bytes(c, touched_experts) + 2.0 * V * H + 2.0 * batch * H
            + batch * keys * kv_per_token)


def prefill_flops(c, layers, n_tokens) -> float:
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, V, K = c["intermediate_size"], c["vocab_size"], c["num_experts_per_tok"]
    per_token = 2.0 * ((Q + 2 * KV) * H + H * Q + 3 * I * H * (1 + K) + c["num_local_experts"] * H)
    attn = 0.0
    for i in range(layers):
        nope = (i + 1) % c["nope_layer_interval"] == 0
        C = c["attention_chunk_size"]
        keys = n_tokens * (n_tokens + 1) / 2 if (nope or C >= n_tokens) else None
        if keys is None:
            full, rem = divmod(n_tokens, C)
            keys = full * C * (C + 1) / 2 + rem * (rem + 1) / 2
        attn += 4.0 * Q * keys
    return layers * per_token * n_tokens + attn + 2.0 * V * H


def prefill_bound_ms(c, layers, n_tokens, n_seqs, pieces, pk) -> float:
    """Milliseconds a prefill of n_seqs prompts of n_tokens would take with every kernel at its own bound: the
    contractions at the tensor peak, except the routed experts, which cannot be faster than reading every
    expert's weights once per piece of the step; the head reads its matrix once."""
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, V, K, E = c["intermediate_size"], c["vocab_size"], c["num_experts_per_tok"], c["num_local_experts"]
    T = n_tokens * n_seqs
    peak, hbm = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    dense = 2.0 * T * ((Q + 2 * KV) * H + H * Q + 3 * I * H + E * H)
    routed_flops = 2.0 * T * K * 3 * I * H
    routed_bytes = 2.0 * min(E, T * K) * 3 * I * H * pieces
    attn = (prefill_flops(c, 1, n_tokens) - 2.0 * V * H - prefill_flops_linear(c, n_tokens)) * n_seqs
    per_layer = (dense + attn) / peak + max(routed_flops / peak, routed_bytes / hbm)
    return 1e3 * (layers * per_layer + 2.0 * V * H / hbm)


def prefill_flops_linear(c, n_tokens) -> float:
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, K = c["intermediate_size"], c["num_experts_per_tok"]
    return 2.0 * ((Q + 2 * KV) * H + H * Q + 3 * I * H * (1 + K) + c["num_local_experts"] * H) * n_tokens


def run(args) -> dict:
    import torch
    from cpi_b200.api import Model
    from cpi_b200.csrc import lib as K
    from cpi_b200.engine import StepEntry

    pk = peaks()
    cfg = dict(SCOUT)
    cfg["num_hidden_layers"] = args.layers
    B, ctx, steps, warm = args.batch, args.context, args.steps, args.warmup
    max_b = max(B, 1 if args.skip_points else 64)
    t0 = time.time()
    model = Model.random(cfg, seed=0, dtype="bfloat16", max_batch=max_b, max_context=ctx, device="cuda:0")
    eng = model.engine
    torch.cuda.synchronize()
    build_s = time.time() - t0
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(1234)

    def toks(n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    out_tok = torch.empty(max_b, dtype=torch.int32, device="cuda:0")

    def timed_decode(batch, n_steps, n_warm, count_experts=True):
        """Prefill `batch` prompts so that the timed steps end at the full context; device-timed.  Returns
        (milliseconds, kernels launched, bytes the timed steps had to read, experts touched per layer and step
        as (mean, least, most))."""
        plen = ctx - (n_steps + n_warm) - 1
        prompts = [toks(plen) for _ in range(batch)]
        feed = [toks(batch) for _ in range(n_steps + n_warm)]

        def start():
            slots = [eng.acquire_slot() for _ in range(batch)]
            eng.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
            return slots

        def one(slots, i):
            lg = eng.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            K.argmax(lg, out_tok[:batch])

        slots = start()
        for i in range(n_warm):
            one(slots, i)
        torch.cuda.synchronize()
        l0 = K.kernel_launches() + eng.graph_kernel_launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_warm, n_warm + n_steps):
            one(slots, i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = K.kernel_launches() + eng.graph_kernel_launches - l0
        for s in slots:
            eng.release_slot(s)
        # the same prompts and the same feed once more, untimed, with the routing recorded: the experts that
        # each of the timed steps touched in each layer
        per_step = []
        if count_experts:
            cap = eng.capture_routing(True)
            slots = start()
            for i in range(n_warm + n_steps):
                for lst in cap.values():
                    lst.clear()
                one(slots, i)
                if i >= n_warm:
                    torch.cuda.synchronize()
                    per_step.append([len(set(lst[0].flatten().tolist())) for lst in cap.values() if lst])
            eng.capture_routing(False)
            for s in slots:
                eng.release_slot(s)
        else:
            per_step = [[min(batch * cfg["num_experts_per_tok"], cfg["num_local_experts"])] * args.layers] * n_steps
        means = [sum(x) / len(x) for x in per_step]
        total_bytes = sum(decode_step_bytes(cfg, args.layers, batch, plen + n_warm + k + 1, m)
                          for k, m in enumerate(means))
        touched = (sum(means) / len(means), min(min(x) for x in per_step), max(max(x) for x in per_step))
        return ms, launches, total_bytes, touched

    def e2e_decode(batch, n_steps, n_warm):
        """The same through `Model.generate`: host token ids in, sampled ids read back every step."""
        plen = ctx - (n_steps + n_warm) - 1
        prompts = [toks(plen) for _ in range(batch)]
        # warm-up: the same batch for `n_warm` steps (it also captures this batch size's decode graph)
        model.generate(prompts, max_new=n_warm + 1, temperature=0.0, stop_ids=[])
        model.generate(prompts, max_new=n_steps + 1, temperature=0.0, stop_ids=[])
        st = model.stats()
        return batch * st.decode_steps / (st.decode_ms / 1e3)

    def timed_prefill(n_seqs, reps):
        times = []
        for r in range(reps + 1):                            # the first pass warms up
            slots = [eng.acquire_slot() for _ in range(n_seqs)]
            entries = [StepEntry(x, toks(pre_n), [pre_n - 1]) for x in slots]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step(entries)
            e1.record()
            torch.cuda.synchronize()
            if r:
                times.append(e0.elapsed_time(e1))
            for x in slots:
                eng.release_slot(x)
        return sorted(times)[len(times) // 2]

    def prefill_record(n_seqs, ms):
        pieces = -(-n_seqs * pre_n // eng.max_step_tokens)
        flops = n_seqs * (prefill_flops(cfg, args.layers, pre_n) - 2.0 * V * cfg["hidden_size"]) \
            + 2.0 * V * cfg["hidden_size"] * n_seqs
        sustained = pk.get("bf16_tflops_sustained")
        return {"value": round(n_seqs * pre_n / (ms / 1e3), 1), "tokens": n_seqs * pre_n, "ms": round(ms, 3),
                "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                # the same against the library product's rate in a seconds-long loop under the power cap: a step
                # of tens of milliseconds runs at those clocks, not at a burst's
                "frac_of_sustained": None if not sustained else round(flops / (ms / 1e3) / (sustained * 1e12), 4),
                "frac_per_kernel": round(prefill_bound_ms(cfg, args.layers, pre_n, n_seqs, pieces, pk) / ms, 4),
                "peak": f"bf16_tflops (burst, {pk['source']})", "tokens_per_piece": min(n_seqs * pre_n, eng.max_step_tokens)}

    # ---- prefill of 2,048 tokens: one sequence, and eight in one call ---------------------------------------
    pre_n = 2048
    pre = timed_prefill(1, 3)
    pre8 = None if args.skip_points else timed_prefill(8, 2)

    # ---- the headline: decode at the given batch ----------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    ms, launches, step_bytes, touched = timed_decode(B, steps, warm)
    clock_rec = clocks.stop()
    value = B * steps / (ms / 1e3)
    achieved = step_bytes / (ms / 1e3) / 1e9

    # ---- end to end through the Python entry point --------------------------------------------------
    e2e_value = e2e_decode(B, steps, warm)
    h2d = eng.stager.bytes_staged
    d2h = B * 4

    points, points_e2e, points_frac = {}, {}, {}
    if not args.skip_points:
        for b in (1, 64):
            k = max(4, steps if b == 1 else steps // 2)          # batch-1 steps are short: time more of them
            w = max(3, warm) + (4 if b == 1 else 0)
            m, _, nbytes, _ = timed_decode(b, k, w, count_experts=b > 1)
            points[f"decode_b{b}"] = round(b * k / (m / 1e3), 2)
            points_frac[f"decode_b{b}"] = round(nbytes / (m / 1e3) / 1e9 / pk["hbm_gbs"], 4)
            points_e2e[f"decode_b{b}"] = round(e2e_decode(b, k, w), 2)

    # ---- where the time goes: phases of one prefill and of one decode step (eager, one stream) ---------
    timer = eng.profile_phases(True)
    for it in range(2):                                      # the first pass warms the eager paths up
        timer.reset()
        s = eng.acquire_slot()
        eng.step([StepEntry(s, toks(pre_n), [pre_n - 1])])
        eng.release_slot(s)
    pre_ph = dict(timer.collect().get("prefill", {}))
    slots = [eng.acquire_slot() for _ in range(B)]
    eng.step([StepEntry(x, toks(ctx - 8), []) for x in slots])
    eng.step([StepEntry(x, toks(1), [0]) for x in slots])
    timer.reset()
    for _ in range(4):
        eng.step([StepEntry(x, toks(1), [0]) for x in slots])
    for x in slots:
        eng.release_slot(x)
    ph = timer.collect()
    eng.profile_phases(False)
    phases = {"prefill_ms": {k: round(v, 3) for k, v in pre_ph.items()},
              "decode_ms": {k: round(v / 4, 3) for k, v in ph.get("decode", {}).items()}}

    return {
        "metric": f"decode tok/s @ batch {B} (Llama4 Scout layer sizes, bf16, random weights)",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
        "impl": "cpi_b200",
        "config": {"model": "llama4-scout-layer-sizes", "layers": args.layers, "layers_full_model": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "experts": cfg["num_local_experts"], "top_k": cfg["num_experts_per_tok"],
                   "expert_inter": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "chunk": cfg["attention_chunk_size"], "nope_interval": cfg["nope_layer_interval"],
                   "global_batch": B, "seq_len": ctx, "decode_context_end": ctx, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (a step reads > 10 GB of weights)",
                   "experts_touched_per_layer": round(touched[0], 2)},
        "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill_record(1, pre),
        "prefill_b8": None if pre8 is None else prefill_record(8, pre8),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "experts_touched": {"mean": round(touched[0], 2), "least": touched[1], "most": touched[2],
                                         "counted": "over the timed steps, in an untimed replay of the same feed"}},
        "points": points,
        "points_e2e": points_e2e,
        "points_roofline_frac": points_frac,
        "phases": phases,
        "clocks": clock_rec,
        "build_s": round(build_s, 1),
    }


def run_workload(args) -> dict:
    """BASELINE's two further workloads through the Python entry point."""
    import random

    import torch
    from cpi_b200.api import Model
    cfg = dict(SCOUT)
    if args.workload == "maverick4":
        cfg.update(num_hidden_layers=4, interleave_moe_layer_step=2, num_local_experts=128)
        cfg["rope_scaling"] = dict(cfg["rope_scaling"], factor=8.0)
        rnd = random.Random(0)
        lens, new = [rnd.randint(64, 2048) for _ in range(32)], 128
    else:
        cfg.update(num_hidden_layers=12)
        lens, new = [131072], 256
    model = Model.random(cfg, seed=0, dtype="bfloat16", max_batch=len(lens), max_context=max(lens) + new + 64,
                         device="cuda:0")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    clocks = ClockSampler()
    for it in range(2):
        if it == 1:
            clocks.start()
        torch.cuda.synchronize()
        t0 = time.time()
        res = model.generate(prompts, max_new=new, temperature=0.0, stop_ids=[])
        torch.cuda.synchronize()
        total = time.time() - t0
    clock_rec = clocks.stop()
    model.engine.check_device_errors()
    st = model.stats()
    n_new = sum(len(r.tokens) for r in res)
    return {"metric": f"tokens/s through Model.generate, workload {args.workload} (bf16, random weights)",
            "value": round((n_new - len(lens)) / (st.decode_ms / 1e3), 1), "unit": "decoded tok/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "bf16", "impl": "cpi_b200",
            "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
            "config": {"model": args.workload, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                       "experts": cfg["num_local_experts"], "moe_layer_step": cfg["interleave_moe_layer_step"],
                       "dense_inter": cfg["intermediate_size_mlp"], "expert_inter": cfg["intermediate_size"],
                       "vocab": cfg["vocab_size"], "prompts": len(lens), "prompt_tokens": sum(lens),
                       "longest_prompt": max(lens), "new_tokens_each": new, "parallelism": "single-gpu"},
            "prefill": {"value": round(sum(lens) / (st.prefill_ms / 1e3), 1), "tokens": sum(lens),
                        "ms": round(st.prefill_ms, 2)},
            "decode": {"steps": st.decode_steps, "ms": round(st.decode_ms, 2),
                       "ms_per_step": round(st.decode_ms / max(st.decode_steps, 1), 3)},
            "total_s": round(total, 3), "device_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1),
            "clocks": clock_rec}


def run_contexts(args) -> dict:
    """Decode at longer contexts and a long single prefill, 12 layers of Scout's sizes: (batch, context) of
    (1, 32768), (8, 32768), (64, 8192), (1, 131072), (8, 131072), and a prefill of one 32,768-token prompt.  Every
    cache is filled by a real prefill; decode steps are device-timed as in the default run; the bytes of a step
    count every weight once (experts by the expected number touched under uniform routing) and the keys and
    values that each layer's window lets through."""
    import torch
    from cpi_b200.api import Model
    from cpi_b200.csrc import lib as K
    from cpi_b200.engine import StepEntry
    pk = peaks()
    cfg = dict(SCOUT)
    L = 12
    cfg["num_hidden_layers"] = L
    V, E = cfg["vocab_size"], cfg["num_local_experts"]
    g = torch.Generator().manual_seed(7)
    out = {"metric": "decode tok/s at longer contexts (12 layers of Llama4 Scout sizes, bf16, random weights)",
           "unit": "tok/s", "n_gpus": 1, "dtype": "bf16", "impl": "cpi_b200", "higher_is_better": True,
           "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
           "config": {"model": "llama4-scout-layer-sizes", "layers": L, "layers_full_model": FULL_LAYERS,
                      "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                      "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "experts": E,
                      "expert_inter": cfg["intermediate_size"], "vocab": V, "chunk": cfg["attention_chunk_size"],
                      "nope_interval": cfg["nope_layer_interval"], "parallelism": "single-gpu"},
           "points": {}, "clocks": None}
    steps, warm = 16, 4
    clocks = ClockSampler()
    clocks.start()
    for batch, ctx in ((1, 32768), (8, 32768), (64, 8192), (1, 131072), (8, 131072)):
        model = Model.random(cfg, seed=0, dtype="bfloat16", max_batch=batch, max_context=ctx + 64, device="cuda:0")
        eng = model.engine
        plen = ctx - steps - warm
        slots = [eng.acquire_slot() for _ in range(batch)]
        for s in slots:                                   # one prompt at a time: the pieces stay 8,192 tokens
            eng.step([StepEntry(s, torch.randint(0, V, (plen,), generator=g).tolist(), [])])
        tok = torch.empty(batch, dtype=torch.int32, device="cuda:0")
        feed = [torch.randint(0, V, (batch,), generator=g).tolist() for _ in range(steps + warm)]

        def one(i):
            lg = eng.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            K.argmax(lg, tok)

        for i in range(warm):
            one(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warm, warm + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        eng.check_device_errors()
        ms = e0.elapsed_time(e1) / steps
        touched = E * (1.0 - (1.0 - 1.0 / E) ** batch)
        nbytes = decode_step_bytes(cfg, L, batch, ctx - steps / 2, touched)
        out["points"][f"decode_b{batch}_ctx{ctx}"] = {
            "tok_s": round(batch / (ms / 1e3), 1), "ms_per_step": round(ms, 3),
            "roofline_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
            "cache_gb_held": round(sum(g_.k.numel() * 2 * 2 for g_ in eng.cache.groups) / 1e9, 1)}
        if (batch, ctx) == (1, 32768):                    # the long single prefill, on the same model
            for s in slots:
                eng.release_slot(s)
            slots = []
            times = []
            for r in range(2):
                s = eng.acquire_slot()
                p = torch.randint(0, V, (32768,), generator=g).tolist()
                e0.record()
                eng.step([StepEntry(s, p, [32767])])
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
                eng.release_slot(s)
            pms = min(times)
            # flops of 12 layers at 32,768 tokens: the linear parts per token, attention by each layer's window
            fl = prefill_flops(cfg, L, 32768)
            out["points"]["prefill_1x32768"] = {"tok_s": round(32768 / (pms / 1e3), 1), "ms": round(pms, 2),
                                                "frac": round(fl / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                                                "peak": f"bf16_tflops (burst, {pk['source']})"}
        for s in slots:
            eng.release_slot(s)
        del model, eng
        torch.cuda.empty_cache()
    out["clocks"] = clocks.stop()
    out["value"] = out["points"]["decode_b8_ctx32768"]["tok_s"]
    return out


def run_cpu_baseline(args) -> dict:
    """Tokens per second on the host's cores at the two tiny configurations inside what the reference's engine
    computes: the reference's own CPU engine (unmodified, compiled with tests/golden/ref_harness.cpp; one
    forward_token call per token, as its generate loop does) and this repository's plain implementation (whole
    sequences, one forward per generated token as its greedy loop does, and one forward over all positions)."""
    import re
    import tempfile
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama4 as P
    import tiny
    golden = os.path.join(ROOT, "tests", "golden")
    ref = args.reference_root
    out = {"metric": "CPU baseline: tok/s at the tiny reference-compatible configurations (float32)", "unit": "tok/s",
           "impl": "cpu_baseline", "n_gpus": 0, "cpu_threads": os.cpu_count(), "points": {}}
    exe = None
    if ref and os.path.isdir(os.path.join(ref, "src", "engine")):
        work = tempfile.mkdtemp(prefix="cpi_cpu_baseline_")
        exe = os.path.join(work, "ref_harness")
        srcs = [os.path.join(ref, p) for p in ("src/engine/llama4_cpu_engine.cpp", "src/model/safetensors_loader.cpp",
                                               "src/platform/mmap_file.cpp")]
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
        r = subprocess.run(["g++", "-std=c++20", "-O2", "-mavx2", "-mfma", "-fopenmp", f"-I{ref}/include",
                            f"-I{cuda_inc}", os.path.join(golden, "ref_harness.cpp"), *srcs, "-o", exe],
                           capture_output=True, text=True)
        if r.returncode != 0:
            out["reference_cpu_engine"] = "does not compile here: " + r.stderr.strip().splitlines()[-1][:200]
            exe = None
    else:
        out["reference_cpu_engine"] = "no checkout given (--reference-root DIR)"
    for name, n_tokens in (("R", 48), ("R2", 70)):
        d = tiny.make_model_dir(name)
        c = tiny.config(name)["text_config"]
        rs = c["rope_scaling"]
        tokens = tiny.random_tokens(n_tokens, c["vocab_size"], 77)
        point = {"tokens": n_tokens, "layers": c["num_hidden_layers"], "hidden": c["hidden_size"]}
        if exe:
            argv = [exe, d, os.path.join(os.path.dirname(exe), f"logits_{name}.f32"), c["vocab_size"],
                    c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                    c["num_hidden_layers"], c["num_local_experts"], c["intermediate_size"], c["intermediate_size"],
                    rs["original_max_position_embeddings"], c["rope_theta"], rs["factor"], rs["low_freq_factor"],
                    rs["high_freq_factor"], *tokens]
            best = None
            for _ in range(3):
                r = subprocess.run([str(a) for a in argv], capture_output=True, text=True, check=True)
                ms = float(re.search(r"forward_ms=([0-9.]+)", r.stderr).group(1))
                best = ms if best is None else min(best, ms)
            point["reference_cpu_engine_tok_s"] = round(n_tokens / (best / 1e3), 1)
        pc, W = P.read_config(d), P.read_weights(d)
        P.forward(pc, W, tokens)
        t0 = time.perf_counter()
        P.forward(pc, W, tokens)
        point["plain_all_positions_tok_s"] = round(n_tokens / (time.perf_counter() - t0), 1)
        t0 = time.perf_counter()
        P.greedy_generate(pc, W, tokens[:n_tokens - 8], 8)
        point["plain_greedy_tok_s"] = round(8 / (time.perf_counter() - t0), 2)
        try:
            import torch
            gpu = torch.cuda.is_available()
        except ImportError:
            gpu = False
        if gpu:                                     # the same model through this library, for scale
            from cpi_b200.api import Model
            for dtype in ("float32", "bfloat16"):
                m = Model.load(d, dtype=dtype, max_batch=1, max_context=256)
                m.generate([tokens[:n_tokens - 8]], max_new=64, temperature=0.0, stop_ids=[])
                m.generate([tokens[:n_tokens - 8]], max_new=64, temperature=0.0, stop_ids=[])
                st = m.stats()
                point[f"cpi_b200_{dtype}_decode_tok_s"] = round(st.decode_steps / (st.decode_ms / 1e3), 1)
        out["points"][name] = point
    return out


def reference_arm_reason() -> str:
    """Why `--impl reference` has nothing to run, as found on this image (one line)."""
    return ("kurulav1/cpi is a CMake C++/CUDA project (no setup.py or pyproject.toml, so pip has nothing to install); "
            "its stock CMake build stops here at the first C++ file: CMakeLists.txt:40 passes '-Wall -Wextra -Wpedantic' "
            "as one unquoted generator expression and g++ gets the option '-Wpedantic>'; and its CUDA engine carries "
            "the 48-layer Scout sizes as compiled-in members (include/engine/llama4_cuda_engine.hpp:121-140) and runs "
            "one sequence, so it could run neither this 24-layer configuration nor a batch of 8 unmodified")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="cpi_b200")
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", choices=["scout24", "maverick4", "long131k", "contexts", "cpu_baseline"],
                    default="scout24")
    ap.add_argument("--reference-root", default=os.environ.get("CPI_REFERENCE_ROOT"),
                    help="a checkout of kurulav1/cpi (for --workload cpu_baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": reference_arm_reason()}))
        return 0
    if args.workload == "cpu_baseline":
        print(json.dumps(run_cpu_baseline(args)))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "cpi_b200 is a single-GPU library: run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload == "contexts":
        print(json.dumps(run_contexts(args)))
        return 0
    print(json.dumps(run(args) if args.workload == "scout24" else run_workload(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
