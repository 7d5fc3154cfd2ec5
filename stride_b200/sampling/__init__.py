"""Sampling: parameters, the seeded host sampler (C++, ``csrc/runtime/sampler.hpp``)
and the device kernel for greedy and temperature draws (``csrc/kernels/sampling.cu``).

Names, defaults and validation are the reference's
(crates/stride-core/src/sampling.rs:5-80): temperature 1.0 in [0, 2] (0 is greedy),
top_p 1.0 in (0, 1], top_k None (>= 1; 1 is greedy), max_tokens 128, min_tokens 0,
stop_tokens [], seed None (the engine then derives one from the request id),
ignore_eos False.
"""

from ..csrc.build import load_runtime
from ..csrc.ops import sample_rows


def SamplingParams(temperature: float = 1.0, top_p: float = 1.0, top_k=None, max_tokens: int = 128, min_tokens: int = 0,
                   stop_tokens=(), seed=None, ignore_eos: bool = False):
    """Validated sampling parameters (raises ValueError on a bad value)."""
    p = load_runtime().SamplingParams(float(temperature), float(top_p), top_k, int(max_tokens), int(min_tokens),
                                      [int(t) for t in stop_tokens], seed, bool(ignore_eos))
    p.validate()
    return p


def greedy(max_tokens: int = 128):
    return load_runtime().SamplingParams.greedy(max_tokens)


def Sampler(params, eos: int = -1, fallback_seed: int = 0):
    return load_runtime().Sampler(params, eos, fallback_seed)


def Rng(seed: int):
    return load_runtime().Rng(seed)


__all__ = ["SamplingParams", "greedy", "Sampler", "Rng", "sample_rows"]
