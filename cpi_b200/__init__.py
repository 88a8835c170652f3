"""cpi_b200: a small model library with generation of its own on one B200."""
from .config import ConfigError, ModelSpec, spec_from_model_dir
from .weights import WeightsError, write_random_model

__all__ = ["ConfigError", "ModelSpec", "spec_from_model_dir", "WeightsError",
           "write_random_model", "Engine", "StepEntry", "Model", "generate"]


def __getattr__(name):
    if name in ("Engine", "StepEntry"):
        from . import engine
        return getattr(engine, name)
    if name in ("Model", "generate", "GenerationResult", "SamplingParams"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
