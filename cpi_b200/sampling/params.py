"""Sampling options, with the reference's names, defaults and meanings.

Reference: temperature `--temp` (default 0.8; <= 0 is greedy), `--top-k` 40, `--top-p` 0.9,
`--repeat-penalty` 1.0, `--no-repeat-ngram` 0 (src/app/main_cli.cpp:217-241,
include/engine/llama_engine.hpp:74-77).  The reference draws from an unseeded generator
(src/engine/llama4_cuda_engine.cu:214); `seed` is this library's addition.
"""
from __future__ import annotations

from dataclasses import dataclass

MAX_TOP_K = 256


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    seed: int = 0

    def validate(self) -> None:
        if self.temperature > 0 and self.top_k > MAX_TOP_K:
            raise ValueError(f"top_k = {self.top_k} is not supported when sampling (at most {MAX_TOP_K}); "
                             "use temperature <= 0 for greedy decoding")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if self.no_repeat_ngram_size < 0:
            raise ValueError(f"no_repeat_ngram_size must be >= 0, got {self.no_repeat_ngram_size}")

    @property
    def is_plain_greedy(self) -> bool:
        """The reference's fast path: arg-max on the device, nothing else
        (src/engine/llama4_cuda_engine.cu:502-515)."""
        return self.temperature <= 0 and self.repetition_penalty <= 1.0 and self.no_repeat_ngram_size <= 1


GREEDY = SamplingParams(temperature=0.0)
