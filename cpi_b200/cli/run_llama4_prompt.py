"""One prompt through a Llama4 model folder, in process: `run_llama4_prompt MODEL_DIR PROMPT`.

The reference's Python entry (tools/run_llama4_prompt.py:36-83) tokenises a chat prompt with the
folder's tokenizer.json, runs the `llama_infer` binary with `--tokens`, reads its "Output tokens:"
line, cuts the answer at the first stop id and decodes it; its options are `model_dir prompt
--binary --system-prompt --max-new (64) --temp (0.0)`.  Here the model runs in this process through
`cpi_b200.api.Model`, and the prompt is token ids ("5,17,3").  Text is taken only when the
`tokenizers` package can be imported and the folder has a tokenizer.json: then the prompt is wrapped
in the same chat frame (system and user turns, the assistant's header open) and the answer is
decoded as well.  The stop ids come from the folder's configuration, or from --stop-ids.
"""
from __future__ import annotations

import argparse
import os
import re
import sys


def chat_frame(system_prompt: str, user_prompt: str) -> str:
    turn = lambda role, text: f"<|header_start|>{role}<|header_end|>\n\n{text}<|eot|>"
    return ("<|begin_of_text|>" + turn("system", system_prompt) + turn("user", user_prompt)
            + "<|header_start|>assistant<|header_end|>\n\n")


def cut_at_stop(tokens, stop_ids) -> list:
    out = []
    for t in tokens:
        if t in stop_ids:
            break
        out.append(t)
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="run_llama4_prompt", description=__doc__.splitlines()[0])
    p.add_argument("model_dir")
    p.add_argument("prompt", help="token ids, comma separated (or text, if the folder has a tokenizer.json "
                                  "and the tokenizers package is installed)")
    p.add_argument("--system-prompt", default="You are a concise helpful assistant.")
    p.add_argument("--max-new", type=int, default=64)
    p.add_argument("--temp", type=float, default=0.0)
    p.add_argument("--stop-ids", default=None, help="comma separated; default: the configuration's eos_token_id")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--max-context", type=int, default=2048)
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(argv)

    tokenizer = None
    if re.fullmatch(r"[\d,\s]+", a.prompt):
        prompt_ids = [int(x) for x in re.split(r"[,\s]+", a.prompt.strip()) if x]
    else:
        path = os.path.join(a.model_dir, "tokenizer.json")
        try:
            from tokenizers import Tokenizer
        except ImportError:
            print("the prompt is text, and the tokenizers package is not installed: give token ids", file=sys.stderr)
            return 1
        if not os.path.exists(path):
            print(f"the prompt is text, and there is no {path}: give token ids", file=sys.stderr)
            return 1
        tokenizer = Tokenizer.from_file(path)
        prompt_ids = tokenizer.encode(chat_frame(a.system_prompt, a.prompt), add_special_tokens=False).ids

    from ..api import Model
    model = Model.load(a.model_dir, dtype=a.dtype, max_batch=1, max_context=a.max_context)
    stops = (list(model.engine.spec.stop_token_ids) if a.stop_ids is None
             else [int(x) for x in a.stop_ids.split(",") if x.strip()])
    res = model.generate([prompt_ids], max_new=a.max_new, temperature=a.temp, seed=a.seed, stop_ids=stops)[0]
    print("Output tokens:" + "".join(f" {t}" for t in prompt_ids + res.tokens))
    answer = cut_at_stop(res.tokens, set(stops))
    print("Answer tokens:" + "".join(f" {t}" for t in answer))
    if tokenizer is not None:
        print("\nDecoded answer:\n" + tokenizer.decode(answer, skip_special_tokens=True).strip())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
