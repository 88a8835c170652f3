"""`llama_infer`-style command line on token ids.

Flags keep the reference's names and meanings where it has them (src/app/main_cli.cpp:195-343):
positional model folder, --tokens, --max-new (16), --temp (0.8), --max-context (2048), --top-k (40),
--top-p (0.9), --repeat-penalty (1.0), --no-repeat-ngram (0), --eos-token (-1 disables),
--inspect-next-topk, --trace-steps, --benchmark, --benchmark-reps, --benchmark-warmup; the
LLAMA_INFER_* environment variables give defaults (:45-80, :190-193).  Output lines: "Output tokens:"
(prompt + generated, src/app/main_modes.cpp:507-513), "[perf]" (:549-559), "[bench]" (:590-606).
Exit codes: 1 argument error, 2 fatal error (src/main.cpp:67, :248).  Text prompts and tokenisers are
outside this library: prompts are token ids.  Added here: --tokens-file, --batch-file, --stop-ids,
--seed, --dtype, --random.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _env(name, cast, default):
    raw = os.environ.get(name)
    if raw is None:
        return default
    try:
        return cast(raw)
    except ValueError:
        raise SystemExit(f"argument error: invalid value for env {name}: {raw}")


def parse_tokens(csv: str) -> list:
    out = []
    for piece in csv.replace("\n", ",").replace(" ", ",").split(","):
        if piece.strip():
            out.append(int(piece))
    return out


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="llama_infer", description="Generate token ids with a Llama4 model folder.")
    p.add_argument("model_dir", nargs="?", help="folder with config.json and *.safetensors")
    p.add_argument("--random", metavar="CONFIG.json", help="draw random weights for this configuration instead")
    p.add_argument("--tokens", default="1,2,3", help="prompt token ids, comma separated")
    p.add_argument("--tokens-file", help="file with the prompt's token ids")
    p.add_argument("--batch-file", help="file with one prompt (comma-separated ids) per line")
    p.add_argument("--max-new", type=int, default=_env("LLAMA_INFER_DEFAULT_MAX_NEW", int, 16))
    p.add_argument("--temp", type=float, default=_env("LLAMA_INFER_DEFAULT_TEMP", float, 0.8))
    p.add_argument("--max-context", type=int, default=_env("LLAMA_INFER_MAX_CONTEXT", int, 2048))
    p.add_argument("--top-k", type=int, default=_env("LLAMA_INFER_TOP_K", int, 40))
    p.add_argument("--top-p", type=float, default=_env("LLAMA_INFER_TOP_P", float, 0.9))
    p.add_argument("--repeat-penalty", type=float, default=_env("LLAMA_INFER_REPEAT_PENALTY", float, 1.0))
    p.add_argument("--no-repeat-ngram", type=int, default=_env("LLAMA_INFER_NO_REPEAT_NGRAM", int, 0))
    p.add_argument("--eos-token", type=int, default=_env("LLAMA_INFER_EOS_TOKEN_ID", int, None),
                   help="end token id; -1 disables stopping; default: the model's own")
    p.add_argument("--stop-ids", default="", help="further stop token ids, comma separated")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32", "bf16", "fp32"], default="bfloat16")
    p.add_argument("--inspect-next-topk", type=int, default=0)
    p.add_argument("--trace-steps", type=int, default=0)
    p.add_argument("--benchmark", action="store_true")
    p.add_argument("--benchmark-reps", type=int, default=1)
    p.add_argument("--benchmark-warmup", type=int, default=0)
    return p


def validate(a) -> None:
    """The reference's checks (src/app/main_cli.cpp:133-180) for the flags kept here."""
    def bad(msg):
        raise SystemExit("argument error: " + msg)
    if not a.model_dir and not a.random:
        bad("a model folder (or --random CONFIG.json) is required")
    if a.max_new < 1:
        bad("--max-new must be >= 1")
    if a.max_context < 1:
        bad("--max-context must be >= 1")
    if a.top_k < 0:
        bad("--top-k must be >= 0")
    if not 0.0 <= a.top_p <= 1.0:
        bad("--top-p must be in [0, 1]")
    if a.repeat_penalty <= 0:
        bad("--repeat-penalty must be > 0")
    if a.no_repeat_ngram < 0:
        bad("--no-repeat-ngram must be >= 0")
    if a.benchmark_reps < 1 or a.benchmark_warmup < 0:
        bad("--benchmark-reps must be >= 1 and --benchmark-warmup >= 0")


def main(argv=None) -> int:
    parser = build_parser()
    try:
        a = parser.parse_args(argv)
        validate(a)
        if a.batch_file:
            with open(a.batch_file) as f:
                prompts = [parse_tokens(line) for line in f if line.strip()]
        elif a.tokens_file:
            with open(a.tokens_file) as f:
                prompts = [parse_tokens(f.read())]
        else:
            prompts = [parse_tokens(a.tokens)]
        extra_stops = parse_tokens(a.stop_ids)
    except SystemExit as e:
        if e.code not in (0, None):
            print(e.code if isinstance(e.code, str) else "argument error", file=sys.stderr)
            return 1
        return 0
    except (ValueError, OSError) as e:
        print(f"argument error: {e}", file=sys.stderr)
        return 1
    try:
        from ..api import Model
        kw = dict(dtype=a.dtype, max_batch=len(prompts), max_context=a.max_context)
        if a.random:
            with open(a.random) as f:
                model = Model.random(json.load(f), a.seed, **kw)
        else:
            model = Model.load(a.model_dir, **kw)
        spec = model.engine.spec
        if a.eos_token is None:
            stops = list(spec.stop_token_ids)
        elif a.eos_token < 0:
            stops = []
        else:
            stops = [a.eos_token]
        stops += extra_stops
        print(f"[info] {spec.architecture} layers={len(spec.layers)} hidden={spec.hidden_size} "
              f"vocab={spec.vocab_size} dtype={a.dtype} prompts={len(prompts)}")
        if a.inspect_next_topk > 0:
            import torch
            lg = model.next_token_logits(prompts[0])
            top = torch.topk(lg, min(a.inspect_next_topk, lg.numel()))
            print(f"Next-token top-{a.inspect_next_topk}:")
            for v, i in zip(top.values.tolist(), top.indices.tolist()):
                print(f"  id={i} logit={v:.4f}")
        if a.trace_steps > 0:
            print("Greedy trace:")
            res = model.generate([prompts[0]], max_new=a.trace_steps, temperature=0.0, stop_ids=[])
            for step, t in enumerate(res[0].tokens):
                print(f"  step={step} choose id={t}")
        gen_kw = dict(max_new=a.max_new, temperature=a.temp, top_k=a.top_k, top_p=a.top_p,
                      repetition_penalty=a.repeat_penalty, no_repeat_ngram_size=a.no_repeat_ngram,
                      seed=a.seed, stop_ids=stops)
        for _ in range(a.benchmark_warmup if a.benchmark else 0):
            model.generate(prompts, **gen_kw)
        reps = a.benchmark_reps if a.benchmark else 1
        tot_ms = pre_ms = dec_ms = 0.0
        for _ in range(reps):
            t0 = time.perf_counter()
            results = model.generate(prompts, **gen_kw)
            tot_ms += (time.perf_counter() - t0) * 1e3
            pre_ms += model.stats().prefill_ms
            dec_ms += model.stats().decode_ms
        for p, r in zip(prompts, results):
            print("Output tokens:" + "".join(f" {t}" for t in list(p) + r.tokens))
        st = model.stats()
        gen = st.generated_tokens
        tot_ms, pre_ms, dec_ms = tot_ms / reps, pre_ms / reps, dec_ms / reps
        print(f"[perf] generated_tokens={gen} elapsed_ms={tot_ms:.2f} tok_per_s={1e3 * gen / max(tot_ms, 1e-9):.2f}")
        if a.benchmark:
            pt = max(st.prompt_tokens - len(prompts), 0)
            print(f"[bench] prefill_tokens={pt} prefill_ms={pre_ms:.2f} "
                  f"prefill_tok_per_s={1e3 * pt / max(pre_ms, 1e-9):.2f} decode_tokens={gen} "
                  f"decode_ms={dec_ms:.2f} decode_tok_per_s={1e3 * gen / max(dec_ms, 1e-9):.2f}")
        return 0
    except Exception as e:                                    # noqa: BLE001  (the reference: catch, print, 2)
        print(f"fatal: {type(e).__name__}: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
