"""`llama_infer`-style command line on token ids.

Flags keep the reference's names and meanings where it has them (src/app/main_cli.cpp:195-343):
positional model folder, --tokens, --max-new (16), --temp (0.8), --max-context (2048), --top-k (40),
--top-p (0.9), --repeat-penalty (1.0), --no-repeat-ngram (0), --eos-token (-1 disables),
--rope-theta, --inspect-next-topk, --trace-steps, --benchmark, --benchmark-reps, --benchmark-warmup,
--benchmark-phases, --interactive; the LLAMA_INFER_* environment variables give defaults (:45-80,
:190-193).  Output lines: "Output tokens:" (prompt + generated, src/app/main_modes.cpp:507-513), "[perf]"
or "[perf-avg]" (:549-559), "[bench]" or "[bench-avg] reps=" (:560-606), "[bench-phase]" or
"[bench-phase-avg]" (:576-617).  Exit codes: 1 argument error, 2 fatal error, 3 another instance is running
(src/main.cpp:51-55, :67, :248): like the reference, a process holds an exclusive lock on the file that
LLAMA_INFER_LOCK_PATH names (default /tmp/llama_infer_single_instance.lock, src/app/main_helpers.cpp:24,
:151-193) from its start to its end.
Text prompts and tokenisers are outside this library: prompts are token ids, so --prompt, --tokenizer
and --stop-text are answered with an argument error that names --tokens and --stop-ids, and --cpu with
a fatal error (there is no CPU path).  --interactive speaks the reference's line-by-line JSON protocol
(src/app/main_modes.cpp:46-270) with token ids in place of text: a request {"id", "tokens", "max_new",
"temp", "stop_ids", "shutdown"}, events "start", "delta" {"tokens": [id]}, "metrics" {"token_index"},
"done" {"tokens", "elapsed_ms", "generated_tokens", "tok_per_s"}, "error" {"error"}.
Added here: --tokens-file, --batch-file, --stop-ids, --seed, --dtype, --random, --dump-logits, --preset and
the options that the registered architectures declare (for instance --rope-pairing, --qk-norm-order,
--qk-norm-scope, --router-gate); they reach the model as config.json keys.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

from ..config.registry import cli_options, cli_presets

PHASES = ("rmsnorm", "qkv", "kv_store", "attention", "wo", "mlp", "moe_router", "moe_expert", "moe_merge", "lm_head")


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
    p = argparse.ArgumentParser(prog="llama_infer", description="Generate token ids with a model folder.")
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
    p.add_argument("--benchmark-phases", action="store_true", help="also time the phases of the decode steps")
    p.add_argument("--preset", choices=sorted(cli_presets()), default=None,
                   help="a named set of config.json keys that an architecture registers")
    for flag, key, kind, text in cli_options():       # what the registered architectures let a command line set
        if isinstance(kind, tuple):
            p.add_argument(flag, dest="cfg_" + key, choices=kind, default=None, help=text)
        else:
            p.add_argument(flag, dest="cfg_" + key, type=kind, default=None, help=text)
    p.add_argument("--dump-logits", metavar="FILE",
                   help="write the logits after each prompt as little-endian float32 [prompts, vocab]")
    p.add_argument("--interactive", action="store_true", help="requests as JSON lines on standard input")
    p.add_argument("--cpu", action="store_true", help=argparse.SUPPRESS)
    for flag in ("--prompt", "--tokenizer", "--stop-text", "--system-prompt"):
        p.add_argument(flag, default=None, help=argparse.SUPPRESS)
    return p


def config_overrides(a) -> dict:
    """The config.json keys that the command line replaces: the preset first, single options over it."""
    out = dict(cli_presets()[a.preset]) if a.preset else {}
    for _flag, key, _kind, _text in cli_options():
        if getattr(a, "cfg_" + key, None) is not None:
            out[key] = getattr(a, "cfg_" + key)
    return out


def validate(a) -> None:
    """The reference's checks (src/app/main_cli.cpp:133-180) for the flags kept here."""
    def bad(msg):
        raise SystemExit("argument error: " + msg)
    if not a.model_dir and not a.random:
        bad("a model folder (or --random CONFIG.json) is required")
    for flag, instead in (("prompt", "--tokens / --tokens-file"), ("tokenizer", "--tokens / --tokens-file"),
                          ("system_prompt", "--tokens / --tokens-file"), ("stop_text", "--stop-ids")):
        if getattr(a, flag) is not None:
            bad(f"--{flag.replace('_', '-')} needs a tokeniser, which this library does not have: give token ids "
                f"with {instead}")
    theta = getattr(a, "cfg_rope_theta", None)
    if theta is not None and not theta > 0:
        bad("--rope-theta must be > 0")
    if a.benchmark_phases or a.benchmark_reps != 1 or a.benchmark_warmup != 0:
        a.benchmark = True                     # as the reference's parser does (src/app/main_cli.cpp:255-265)
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


class SingleInstance:
    """The reference's guard (src/app/main_helpers.cpp:151-193): an exclusive, non-blocking lock on a file,
    held while the process runs.  `acquire` answers False when another process holds it (or the file cannot
    be opened), as the reference's does."""

    def __init__(self, path=None):
        self.path = path or os.environ.get("LLAMA_INFER_LOCK_PATH") or "/tmp/llama_infer_single_instance.lock"
        self._fd = None

    def acquire(self) -> bool:
        import fcntl
        try:
            fd = os.open(self.path, os.O_CREAT | os.O_RDWR, 0o644)
        except OSError:
            return False
        try:
            fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except OSError:
            os.close(fd)
            return False
        self._fd = fd
        return True

    def release(self) -> None:
        if self._fd is not None:
            import fcntl
            fcntl.flock(self._fd, fcntl.LOCK_UN)
            os.close(self._fd)
            self._fd = None


def main(argv=None) -> int:
    guard = SingleInstance()
    if not guard.acquire():
        print("Another llama_infer instance is already running.", file=sys.stderr)
        return 3
    try:
        return _main(argv)
    finally:
        guard.release()


def _main(argv=None) -> int:
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
        if a.cpu:
            raise RuntimeError("--cpu: this library has no CPU path; the model runs on its CUDA kernels only")
        from ..api import Model
        kw = dict(dtype=a.dtype, max_batch=len(prompts), max_context=a.max_context,
                  config_overrides=config_overrides(a))
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
        gen_kw = dict(max_new=a.max_new, temperature=a.temp, top_k=a.top_k, top_p=a.top_p,
                      repetition_penalty=a.repeat_penalty, no_repeat_ngram_size=a.no_repeat_ngram,
                      seed=a.seed, stop_ids=stops)
        if a.interactive:
            return interactive(model, gen_kw, sys.stdin, sys.stdout)
        print(f"[info] {spec.architecture} layers={len(spec.layers)} hidden={spec.hidden_size} "
              f"vocab={spec.vocab_size} dtype={a.dtype} prompts={len(prompts)}")
        if a.dump_logits:
            import numpy as np
            rows = [model.next_token_logits(p).float().cpu().numpy() for p in prompts]
            np.stack(rows).astype("<f4").tofile(a.dump_logits)
            print(f"[info] logits after {len(rows)} prompt(s) written to {a.dump_logits}")
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
        for _ in range(a.benchmark_warmup if a.benchmark else 0):
            model.generate(prompts, **gen_kw)
        reps = a.benchmark_reps if a.benchmark else 1
        repeated = a.benchmark and (a.benchmark_reps > 1 or a.benchmark_warmup > 0)
        tot_ms = pre_ms = dec_ms = 0.0
        gen = 0
        for _ in range(reps):
            t0 = time.perf_counter()
            results = model.generate(prompts, **gen_kw)
            tot_ms += (time.perf_counter() - t0) * 1e3
            pre_ms += model.stats().prefill_ms
            dec_ms += model.stats().decode_ms
            gen += model.stats().generated_tokens
        for p, r in zip(prompts, results):
            print("Output tokens:" + "".join(f" {t}" for t in list(p) + r.tokens))
        st = model.stats()
        gen, tot_ms, pre_ms, dec_ms = gen // reps, tot_ms / reps, pre_ms / reps, dec_ms / reps
        rate = lambda n, ms: 1e3 * n / ms if n > 0 and ms > 0 else 0.0
        print(f"[perf{'-avg' if repeated else ''}] generated_tokens={gen} elapsed_ms={tot_ms:.2f} "
              f"tok_per_s={rate(gen, tot_ms):.2f}")
        if a.benchmark:
            pt = max(st.prompt_tokens - len(prompts), 0)
            line = (f"prefill_tokens={pt} prefill_ms={pre_ms:.2f} prefill_tok_per_s={rate(pt, pre_ms):.2f} "
                    f"decode_tokens={gen} decode_ms={dec_ms:.2f} decode_tok_per_s={rate(gen, dec_ms):.2f}")
            if repeated:
                print(f"[bench-avg] reps={reps} {line} total_ms={tot_ms:.2f} total_tok_per_s={rate(gen, tot_ms):.2f}")
            else:
                print(f"[bench] {line}")
        if a.benchmark_phases:
            # a run of its own: with the phase brackets on, steps run eagerly and on one stream, which
            # must not disturb the figures above
            timer = model.engine.profile_phases(True)
            try:
                for _ in range(reps):
                    model.generate(prompts, **gen_kw)
                ms = timer.collect().get("decode", {})
            finally:
                model.engine.profile_phases(False)
            print(f"[bench-phase{'-avg' if repeated else ''}]"
                  + "".join(f" {name}_ms={ms.get(name, 0.0) / reps:.2f}" for name in PHASES))
        return 0
    except Exception as e:                                    # noqa: BLE001  (the reference: catch, print, 2)
        print(f"fatal: {type(e).__name__}: {e}", file=sys.stderr)
        return 2


def interactive(model, defaults: dict, inp, out) -> int:
    """Requests as JSON lines, answered with event lines (src/app/main_modes.cpp:46-270), on token ids."""
    def event(kind, rid, **extra):
        body = {"type": kind}
        if rid:
            body["id"] = rid
        body.update(extra)
        out.write(json.dumps(body, separators=(",", ":")) + "\n")
        out.flush()

    for line in inp:
        line = line.strip()
        if not line:
            continue
        rid = ""
        try:
            req = json.loads(line)
            if not isinstance(req, dict):
                raise ValueError("a request is a JSON object")
            rid = str(req.get("id", ""))
            if req.get("shutdown", False):
                event("done", rid, tokens=[], elapsed_ms=0)
                break
            tokens = req.get("tokens")
            if not isinstance(tokens, list) or not tokens:
                raise ValueError("interactive request missing 'tokens'")
            kw = dict(defaults)
            kw["max_new"] = max(1, int(req.get("max_new", defaults["max_new"])))
            kw["temperature"] = max(0.0, float(req.get("temp", defaults["temperature"])))
            if "stop_ids" in req:
                kw["stop_ids"] = [int(t) for t in req["stop_ids"]]
            stops = set(kw["stop_ids"] or ())
            sent = []

            def on_token(_request, token):
                # a stop token ends the answer and is not part of it (:196-199)
                if token in stops:
                    return False
                sent.append(int(token))
                event("delta", rid, tokens=[int(token)])
                event("metrics", rid, metrics={"token_index": len(sent)})
                return True

            t0 = time.perf_counter()
            event("start", rid)
            model.generate([[int(t) for t in tokens]], on_token=on_token, **kw)
            ms = int((time.perf_counter() - t0) * 1e3)
            event("done", rid, tokens=sent, elapsed_ms=ms, generated_tokens=len(sent),
                  tok_per_s=round(1e3 * len(sent) / ms, 2) if ms > 0 and sent else 0.0)
        except Exception as e:                                # noqa: BLE001  (an error event, and on to the next line)
            event("error", rid, error=f"{type(e).__name__}: {e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
