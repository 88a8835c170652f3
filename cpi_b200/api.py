"""Python entry point: load a model folder (or draw random weights) and generate.

The reference's Python entry is a script that tokenises, spawns the `llama_infer` binary with
`--tokens`, and parses its "Output tokens:" line (tools/run_llama4_prompt.py:36-83); its options are
`model_dir prompt --max-new --temp`.  Here the same call runs in process on token ids:

    model = Model.load(model_dir, dtype="bfloat16", max_batch=8, max_context=2048)
    results = model.generate([[1, 2, 3], [4, 5]], max_new=16, temperature=0.0)
    results[0].tokens, results[0].finish_reason
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

from .engine import Engine, GenerationRequest, GenerationResult, Generator, StepEntry
from .sampling import SamplingParams
from .sampling.sampler import Sampler

__all__ = ["Model", "generate", "GenerationResult", "SamplingParams"]


class Model:
    def __init__(self, engine: Engine, max_batch: int, max_context: Optional[int] = None):
        self.engine = engine
        self.max_batch = max_batch
        self.sampler = Sampler(engine.device, engine.spec.vocab_size)
        self.generator = Generator(engine, self.sampler, max_batch=max_batch,
                                   default_stop_ids=engine.spec.stop_token_ids,
                                   bos_token_id=engine.spec.bos_token_id, max_context=max_context)

    # ---- construction ----------------------------------------------------------------------------
    @staticmethod
    def _cache_args(max_batch, max_context, max_tokens, page_size):
        per_seq = -(-max_context // page_size) * page_size
        return dict(max_tokens=max_tokens if max_tokens is not None else per_seq * max_batch,
                    max_seqs=max_batch, max_seq_len=per_seq, page_size=page_size)

    @classmethod
    def load(cls, model_dir: str, *, dtype="bfloat16", max_batch: int = 1, max_context: int = 2048,
             max_tokens: Optional[int] = None, device="cuda:0", page_size: int = 64,
             config_overrides: Optional[dict] = None) -> "Model":
        """`max_batch` sequences of up to `max_context` positions each (the reference's EngineOptions
        names, include/engine/llama_engine.hpp:67-68); `max_tokens` bounds the cache instead when given.
        The cache is sized in whole pages, but generation keeps to `max_context` itself: a longer prompt
        is an error and a sequence ends when it reaches it.
        `config_overrides`: config.json keys that replace the file's, e.g. {"rope_theta": 1e6} or a
        preset of `cpi_b200.config.registry.cli_presets()`."""
        eng = Engine.from_model_dir(model_dir, config_overrides, dtype=dtype, device=device,
                                    **cls._cache_args(max_batch, max_context, max_tokens, page_size))
        return cls(eng, max_batch, max_context)

    @classmethod
    def random(cls, config_json: dict, seed: int = 0, *, dtype="bfloat16", max_batch: int = 1,
               max_context: int = 2048, max_tokens: Optional[int] = None, device="cuda:0",
               page_size: int = 64, config_overrides: Optional[dict] = None) -> "Model":
        eng = Engine.from_random(config_json, seed, config_overrides, dtype=dtype, device=device,
                                 **cls._cache_args(max_batch, max_context, max_tokens, page_size))
        return cls(eng, max_batch, max_context)

    # ---- use -------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new: int = 16, temperature: float = 0.8,
                 top_k: int = 40, top_p: float = 0.9, repetition_penalty: float = 1.0,
                 no_repeat_ngram_size: int = 0, seed: int = 0, stop_ids: Optional[Sequence[int]] = None,
                 on_token: Optional[Callable[[int, int], bool]] = None) -> list:
        """Generates for every prompt (lists of token ids); returns a GenerationResult per prompt."""
        sp = SamplingParams(temperature, top_k, top_p, repetition_penalty, no_repeat_ngram_size, seed)
        reqs = [GenerationRequest(p, max_new, sp, stop_ids) for p in prompts]
        return self.generator.generate(reqs, on_token)

    def generate_requests(self, requests: Sequence[GenerationRequest], on_token=None) -> list:
        """The same for requests that each bring their own length, sampling parameters and stop ids."""
        return self.generator.generate(requests, on_token)

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], logits="last"):
        """One step of the engine on sequences that the caller manages: `slots` from `acquire_slot()`,
        `tokens[i]` the next tokens of slot i (all prompts, or one token each).  `logits`: "last" (one row per
        sequence), "all", or a list of places per sequence.  Returns float32 logits [rows, vocab] on the
        device, valid until the next step.  Give slots back with `release_slot()`.  What a kernel flags (a token
        id outside the vocabulary, a wait that ran out) is raised by the next step or by
        `engine.check_device_errors()`, which waits for the device."""
        if logits == "last":
            want = [[len(t) - 1] for t in tokens]
        elif logits == "all":
            want = [list(range(len(t))) for t in tokens]
        else:
            want = [list(w) for w in logits]
        return self.engine.step([StepEntry(int(s), list(t), w) for s, t, w in zip(slots, tokens, want)])

    def acquire_slot(self) -> int:
        return self.engine.acquire_slot()

    def release_slot(self, slot: int) -> None:
        self.engine.release_slot(slot)

    def next_token_logits(self, prompt: Sequence[int]):
        """Float32 logits [vocab] after the prompt (the reference's inspect_next_logits,
        src/engine/llama4_cuda_engine.cu:623-674, without its top-k cut)."""
        s = self.engine.acquire_slot()
        try:
            row = self.engine.step([StepEntry(s, list(prompt), [len(prompt) - 1])])[0].clone()
            self.engine.check_device_errors()
            return row
        finally:
            self.engine.release_slot(s)

    def stats(self):
        return self.generator.stats


def generate(model_dir: str, prompts, **kw) -> list:
    """One call: load `model_dir` and generate for `prompts`."""
    load_kw = {k: kw.pop(k) for k in ("dtype", "max_context", "device") if k in kw}
    m = Model.load(model_dir, max_batch=max(1, len(prompts)), **load_kw)
    return m.generate(prompts, **kw)
