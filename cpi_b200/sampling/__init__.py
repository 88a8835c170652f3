from .params import SamplingParams, GREEDY, MAX_TOP_K


def __getattr__(name):
    if name in ("Sampler", "banned_by_ngram", "uniform_for"):
        from . import sampler
        return getattr(sampler, name)
    raise AttributeError(name)
