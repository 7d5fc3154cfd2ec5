"""The host sampler and generator against the plain restatement (no GPU)."""

import numpy as np
import pytest
import torch

import plain_llama as plain
from stride_b200.sampling import Rng, Sampler, SamplingParams, greedy


def test_generator_matches_the_plain_one():
    for seed in (0, 1, 42, 2**63 + 5, 2**64 - 1):
        a, b = Rng(seed), plain.XorShiftRng(seed)
        assert [a.next_u64() for _ in range(20)] == [b.next_u64() for _ in range(20)]
        assert [a.next_f32() for _ in range(20)] == [b.next_f32() for _ in range(20)]


def test_parameter_defaults_and_validation():
    p = SamplingParams()
    assert (p.temperature, p.top_p, p.top_k, p.max_tokens, p.min_tokens, p.stop_tokens, p.seed, p.ignore_eos) == \
        (1.0, 1.0, None, 128, 0, [], None, False)
    assert greedy(5).is_greedy() and SamplingParams(top_k=1).is_greedy() and not SamplingParams().is_greedy()
    assert SamplingParams(top_p=0.9).needs_ranking() and not SamplingParams(temperature=0.5).needs_ranking()
    for bad in (dict(temperature=-0.1), dict(temperature=2.5), dict(temperature=float("nan")), dict(top_p=0.0),
                dict(top_p=1.5), dict(top_k=0), dict(max_tokens=0), dict(min_tokens=9, max_tokens=3)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


@pytest.mark.parametrize("kwargs", [dict(temperature=0.0), dict(temperature=1.0), dict(temperature=0.7, top_k=5),
                                    dict(temperature=1.3, top_p=0.8), dict(top_k=3, top_p=0.5), dict(top_k=1)])
def test_sampler_follows_the_reference_rules(kwargs):
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(8, 301, generator=g) * 2
    s = Sampler(SamplingParams(seed=11, **kwargs), eos=4, fallback_seed=99)
    rng = plain.XorShiftRng(11)
    for row in logits:
        want = plain.sample(row, rng, temperature=kwargs.get("temperature", 1.0), top_k=kwargs.get("top_k"),
                            top_p=kwargs.get("top_p", 1.0))
        assert s.sample(row.numpy(), 0) == want
    assert s.effective_seed == 11 and Sampler(SamplingParams(), 4, 99).effective_seed == 99


@pytest.mark.parametrize("top_k,top_p", [(None, 0.95), (None, 0.3), (50, 1.0), (700, 0.99), (None, 0.999), (40000, 1.0), (1, 0.5)])
def test_the_head_of_the_ranking_is_that_of_a_stable_sort(top_k, top_p):
    """The sampler selects and sorts only the head of the ranking (the first 256 entries, then eight times as many,
    as far as the nucleus reaches). Against a stable sort of the whole vocabulary with the same float32 sums: flat
    rows whose nucleus holds most of the vocabulary, peaked rows, coarse weights with many ties (ties go by
    vocabulary order, also across the edge of a head), all equal."""
    from stride_b200.csrc.build import load_runtime
    rank_head = load_runtime().rank_head
    g = torch.Generator().manual_seed(5)
    n = 30011
    rows = [torch.softmax(torch.randn(n, generator=g) * 0.3, 0), torch.softmax(torch.randn(n, generator=g) * 6, 0),
            torch.softmax(torch.round(torch.randn(n, generator=g) * 2) / 2, 0), torch.full((n,), 1.0 / n),
            torch.softmax(torch.cat([torch.full((300,), 3.0), torch.zeros(n - 300)]), 0)]
    for row in rows:
        w = row.numpy().astype(np.float32)
        order = np.argsort(-w, kind="stable")
        limit = n if top_k is None else min(n, top_k)
        keep = limit
        if top_p < 1.0:
            sums = np.cumsum(w[order], dtype=np.float32)          # sequential float32 additions, as the sampler's
            reached = np.nonzero(sums >= np.float32(top_p))[0]
            nucleus = int(reached[0]) + 1 if len(reached) else n
            keep = min(limit, max(nucleus, 1))
        got = rank_head(w, top_k, top_p)
        assert len(got) == keep, f"keeps {len(got)} tokens, a full sort keeps {keep}"
        assert np.array_equal(np.asarray(got), order[:keep]), "the kept ranking differs from a stable sort's"


def test_eos_suppression_stop_tokens_and_extremes():
    logits = np.array([0.0, 5.0, 1.0, 4.0], dtype=np.float32)
    s = Sampler(SamplingParams(temperature=0.0, min_tokens=2, max_tokens=4, stop_tokens=[3]), eos=1, fallback_seed=0)
    assert s.sample(logits, 0) == 3 and s.sample(logits, 1) == 3 and s.sample(logits, 2) == 1
    assert s.suppressed_token(1) == 1 and s.suppressed_token(2) == -1
    assert s.is_stop(1) and s.is_stop(3) and not s.is_stop(2)
    assert not Sampler(SamplingParams(ignore_eos=True), 1, 0).is_stop(1)
    assert not Sampler(SamplingParams(), -1, 0).is_stop(-1)
    huge = np.array([1e30, -1e30, 3e38], dtype=np.float32)
    assert Sampler(SamplingParams(), -1, 1).sample(huge, 0) == 2
    all_inf = np.full(5, -np.inf, dtype=np.float32)
    assert 0 <= Sampler(SamplingParams(), -1, 1).sample(all_inf, 0) < 5
    with pytest.raises(ValueError):
        Sampler(SamplingParams(), -1, 1).sample(np.zeros(0, dtype=np.float32), 0)


def test_draws_follow_the_distribution_and_a_seed_fixes_the_stream():
    logits = np.log(np.array([0.1, 0.6, 0.3], dtype=np.float32))
    s = Sampler(SamplingParams(seed=5), -1, 0)
    counts = np.bincount([s.sample(logits, 0) for _ in range(20000)], minlength=3) / 20000
    assert np.abs(counts - [0.1, 0.6, 0.3]).max() < 0.02
    a = Sampler(SamplingParams(seed=8), -1, 0)
    b = Sampler(SamplingParams(seed=8), -1, 0)
    assert [a.sample(logits, 0) for _ in range(50)] == [b.sample(logits, 0) for _ in range(50)]
