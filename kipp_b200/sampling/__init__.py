from .params import RECENT_WINDOW, SamplingParams, next_uniform, xorshift64_star

__all__ = ["RECENT_WINDOW", "SamplingParams", "next_uniform", "xorshift64_star", "Sampler"]


def __getattr__(name):
    if name == "Sampler":          # needs torch + the kernels; keep params importable alone
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
