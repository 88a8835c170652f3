"""Decode and prefill throughput of the Llama4 Scout-sized model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch 8] [--context 4096]
    python bench.py --workload maverick4 | long131k      (two further workloads, a JSON line of their own)

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  `value` is decoded tokens per
second, timed on the device with CUDA events around exactly K engine steps (host token ids in, arg-max
on the device); `e2e` is the same through the Python entry point (`Model.generate`), with every
step's token ids copied from pinned host memory and the sampled ids read back.  Between timed
iterations nothing is flushed: one decode step reads tens of GB of weights, far more than the L2 holds.
For N > 1 GPUs it prints one line that says the library is single-GPU and exits with 2.
`phases` holds device milliseconds per phase of one prefill of 2,048 tokens and of one decode step, taken
after everything else with the steps run eagerly on one stream (so their sum exceeds the step times above).

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
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
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
    """Bytes one decode step has to read: every weight it uses once and the cache of the live requests."""
    H, V = c["hidden_size"], c["vocab_size"]
    kv_per_token = 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    return (layers * layer_weight_bytes(c, touched_experts) + 2.0 * V * H + 2.0 * batch * H
            + layers * batch * context * kv_per_token)


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

    def timed_decode(batch, n_steps, n_warm):
        """Prefill `batch` prompts so that the timed steps end at the full context; device-timed."""
        plen = ctx - (n_steps + n_warm) - 1
        slots = [eng.acquire_slot() for _ in range(batch)]
        eng.step([StepEntry(s, toks(plen), []) for s in slots])
        feed = [toks(batch) for _ in range(n_steps + n_warm + 1)]

        def one(i):
            lg = eng.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            K.argmax(lg, out_tok[:batch])

        for i in range(n_warm):
            one(i)
        torch.cuda.synchronize()
        l0 = K.kernel_launches() + eng.graph_kernel_launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_warm, n_warm + n_steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = K.kernel_launches() + eng.graph_kernel_launches - l0
        cap = eng.capture_routing(True)          # one more, untimed, step: how many experts a step touches
        one(n_warm + n_steps)
        torch.cuda.synchronize()
        touched = [len(set(lst[0].flatten().tolist())) for lst in cap.values() if lst]
        eng.capture_routing(False)
        for s in slots:
            eng.release_slot(s)
        return ms, launches, (sum(touched) / len(touched) if touched else 0.0)

    # ---- prefill of 2,048 tokens, one sequence ------------------------------------------------------
    pre_n = 2048
    s = eng.acquire_slot()
    eng.step([StepEntry(s, toks(pre_n), [pre_n - 1])])
    eng.release_slot(s)
    torch.cuda.synchronize()
    pre_ms = []
    for _ in range(3):
        s = eng.acquire_slot()
        p = toks(pre_n)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([StepEntry(s, p, [pre_n - 1])])
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        eng.release_slot(s)
    pre = sorted(pre_ms)[len(pre_ms) // 2]
    pf = prefill_flops(cfg, args.layers, pre_n)

    # ---- the headline: decode at the given batch ----------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    ms, launches, touched = timed_decode(B, steps, warm)
    clock_rec = clocks.stop()
    value = B * steps / (ms / 1e3)
    step_bytes = decode_step_bytes(cfg, args.layers, B, ctx - steps / 2, touched)
    achieved = step_bytes / (ms / steps / 1e3) / 1e9

    # ---- end to end through the Python entry point --------------------------------------------------
    plen = ctx - (steps + warm) - 1
    prompts = [toks(plen) for _ in range(B)]
    # warm-up: the same batch for `warm` steps (it also captures this batch size's decode graph), then the timed run
    model.generate(prompts, max_new=warm + 1, temperature=0.0, stop_ids=[])
    model.generate(prompts, max_new=steps + 1, temperature=0.0, stop_ids=[])
    st = model.stats()
    e2e_value = B * st.decode_steps / (st.decode_ms / 1e3)
    h2d = eng.stager.bytes_staged
    d2h = B * 4

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            k = max(4, steps if b == 1 else steps // 2)          # batch-1 steps are short: time more of them
            m, _, _ = timed_decode(b, k, max(3, warm) + (4 if b == 1 else 0))
            points[f"decode_b{b}"] = round(b * k / (m / 1e3), 2)

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
        "metric": "decode tok/s @ batch 8 (Llama4 Scout layer sizes, bf16, random weights)",
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
                   "experts_touched_per_layer": round(touched, 2)},
        "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(pre_n / (pre / 1e3), 1), "tokens": pre_n, "ms": round(pre, 3),
                    "frac": round(pf / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
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
    ap.add_argument("--workload", choices=["scout24", "maverick4", "long131k"], default="scout24")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "kurulav1/cpi is a CMake C++/CUDA project with neither setup.py nor pyproject.toml: "
                          "pip cannot install it offline (Directory is not installable)"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "cpi_b200 is a single-GPU library: run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    args.warmup = max(args.warmup, 3)
    print(json.dumps(run(args) if args.workload == "scout24" else run_workload(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
