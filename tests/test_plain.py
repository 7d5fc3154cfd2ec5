"""The plain implementation against the reference project's own model code
(golden logits written by tests/golden/make_golden.py) and against itself."""

import os

import numpy as np
import pytest
import torch

import plain_llama as plain
from helpers import TINY, compare_logits, seeded_biases, seeded_state, seeded_tokens

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
GOLDEN_SEED = {"A": 11, "B": 22, "C": 33, "A_bias": 44}
GOLDEN_TOKENS = {"A": 40, "B": 90, "C": 37, "A_bias": 40}


@pytest.mark.parametrize("name", ["A", "B", "C", "A_bias"])
def test_plain_matches_reference_model(name):
    cfg = TINY[name.split("_")[0]]
    state = seeded_state(cfg, GOLDEN_SEED[name])
    if name.endswith("_bias"):      # a checkpoint with q/k/v biases: the reference adds them because the tensors are there
        state.update(seeded_biases(cfg, GOLDEN_SEED[name] + 2))
    tokens = seeded_tokens(GOLDEN_TOKENS[name], cfg["vocab_size"], GOLDEN_SEED[name] + 1)
    want = torch.from_numpy(np.load(os.path.join(GOLDEN, f"tiny_{name}.npy")))
    got = plain.forward(cfg, state, tokens, torch.float32)
    ok, msg = compare_logits(got, want, "float32")
    assert ok, msg
    got64 = plain.forward(cfg, state, tokens, torch.float64)
    ok, msg = compare_logits(got64, want, "float32")
    assert ok, msg


def test_a_prefix_of_the_sequence_gives_the_same_logits():
    cfg = TINY["B"]
    state = seeded_state(cfg, 5)
    tokens = seeded_tokens(50, cfg["vocab_size"], 6)
    whole = plain.forward(cfg, state, tokens, torch.float64)
    part = plain.forward(cfg, state, tokens[:17], torch.float64)
    assert torch.allclose(whole[:17], part, atol=1e-12)


def test_llama3_bands_are_all_in_play_in_tiny_b():
    cfg = TINY["B"]
    plain_freq = plain.rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], None)
    scaled = plain.rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    ratio = scaled / plain_freq
    assert (ratio == 1.0).any(), "no untouched band"
    assert torch.isclose(ratio, torch.tensor(1 / 8.0)).any(), "no fully scaled band"
    assert ((ratio > 1 / 8.0 + 1e-6) & (ratio < 1 - 1e-6)).any(), "no interpolated band"
    legacy = dict(cfg["rope_scaling"])
    legacy["type"] = legacy.pop("rope_type")
    assert torch.equal(plain.rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], legacy), scaled)


def test_window_limits_the_keys():
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 2, 16), torch.randn(9, 1, 16), torch.randn(9, 1, 16)
    full = plain.causal_attention(q, k, v, 0.25)
    win = plain.causal_attention(q, k, v, 0.25, window=3)
    assert torch.allclose(full[:3], win[:3])
    assert not torch.allclose(full[5], win[5])
    alone = plain.causal_attention(q[3:6], k[3:6], v[3:6], 0.25)
    assert torch.allclose(win[5], alone[2], atol=1e-6)


def test_rng_and_sampling_follow_the_reference_rules():
    rng = plain.XorShiftRng(0)
    draws = [rng.next_f32() for _ in range(1000)]
    assert all(0.0 <= d < 1.0 for d in draws) and len(set(draws)) > 990
    assert plain.XorShiftRng(7).next_u64() == plain.XorShiftRng(7).next_u64()
    logits = torch.tensor([0.0, 3.0, 3.0, -1.0])
    assert plain.argmax(logits) == 1
    assert plain.sample(logits, plain.XorShiftRng(1), temperature=0.0) == 1
    assert plain.sample(logits, plain.XorShiftRng(1), temperature=1.0, top_k=1) == 1
    # EOS is suppressed below min_tokens
    assert plain.sample(logits, plain.XorShiftRng(1), temperature=0.0, eos=1, min_tokens=2, generated=0) == 2
    # nucleus 0.5 over probabilities (.64, .24, .12) keeps only the first
    probs = torch.log(torch.tensor([0.12, 0.64, 0.24]))
    assert {plain.sample(probs, plain.XorShiftRng(s), top_p=0.5) for s in range(50)} == {1}
    assert {plain.sample(probs, plain.XorShiftRng(s), top_k=2) for s in range(200)} == {1, 2}
    counts = [0, 0, 0]
    rng = plain.XorShiftRng(3)
    for _ in range(20000):
        counts[plain.sample(probs, rng)] += 1
    for c, p in zip(counts, (0.12, 0.64, 0.24)):
        assert abs(c / 20000 - p) < 0.02
    assert plain.softmax(torch.full((4,), float("-inf"))).tolist() == [0.25] * 4


def test_prefix_chain_values():
    # Values follow from the FNV-1a rules of crates/stride-kvcache/src/hash.rs.
    assert plain._fnv1a(plain.FNV_OFFSET, b"acme") == 0x0724D383F4F6DE0F
    chain = plain.prefix_chain("acme", list(range(32)), 16)
    assert chain == [0xBF0700EAC0C3E9F1, 0x7B8B4746D9BC7AD4]
    assert plain.prefix_chain("acme", list(range(31)), 16) == chain[:1]
    assert plain.prefix_chain("other", list(range(32)), 16)[0] != chain[0]
