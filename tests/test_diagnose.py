"""The equivalence measures in both directions, and negative controls: every comparison that the suite relies on
must be able to fail. Broken variants of the plain implementation (in the manner of
python/stride_worker/autotune/negative_control.py:25-195 and python/tests/test_equivalence.py) are rejected, the
plain implementation itself and rounding-sized noise are accepted. No GPU."""

import pytest
import torch

import plain_llama as plain
from helpers import TINY, compare_logits as suite_compare, seeded_state, seeded_tokens
from stride_b200.diagnose import (COSINE_FLOOR, DECISIVE_GAP, Agreement, compare_logits, first_divergence, report)
from stride_b200.diagnose.prefill import seeded_prompt


def _logits(rows=64, vocab=300, seed=0):
    return torch.randn(rows, vocab, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * 3.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, "float32", "bfloat16"])
def test_identical_logits_are_equivalent_under_every_floor(dtype):
    a = _logits().float()
    agreement = compare_logits(a, a.clone())
    ok, why = agreement.verdict(dtype)
    assert ok, why
    assert agreement.cosine >= max(COSINE_FLOOR.values()) and agreement.argmax_match_rate == 1.0
    assert agreement.top5_overlap == 1.0 and agreement.max_abs_diff == 0.0 and agreement.positions == 64


def test_rounding_sized_noise_passes_and_a_structural_change_fails():
    a = _logits()
    noisy = a + 1e-5 * torch.randn(a.shape, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    assert compare_logits(noisy, a).verdict(torch.float32)[0]
    shifted = torch.roll(a, 1, dims=-1)                  # every row ranks other tokens
    ok, why = compare_logits(shifted, a).verdict(torch.bfloat16)
    assert not ok and "cosine" in why
    bf16_noise = a + 0.02 * torch.randn(a.shape, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    assert compare_logits(bf16_noise, a).verdict(torch.bfloat16)[0]
    assert not compare_logits(bf16_noise, a).verdict(torch.float32)[0], "the float32 floor must not take bfloat16-sized noise"


def test_a_near_tie_that_falls_the_other_way_is_tolerated_and_a_decisive_one_is_not():
    a = _logits(rows=100, vocab=2000).clamp(max=5.0)
    top = a.argmax(-1)
    rows = torch.arange(100)
    a[rows, top] = 10.0
    runner_up = (top + 1) % a.shape[-1]
    a[rows, runner_up] = 10.0 - 0.01                      # every position is a near-tie
    b = a.clone()
    b[rows, runner_up] = 10.0 + 0.01                      # the candidate ranks the other token first everywhere
    agreement = compare_logits(b, a)
    assert agreement.argmax_match_rate == 0.0 and agreement.decisive_disagreement_rate == 0.0
    assert agreement.worst_disagreement_gap == pytest.approx(0.01, abs=1e-9)
    assert agreement.verdict(torch.bfloat16)[0], "disagreements at ties are not counted"
    # now two of a hundred positions disagree although the reference leads by far more than the decisive gap
    c = a.clone()
    a2 = a.clone()
    a2[rows, runner_up] = 10.0 - 1.0
    c[rows, runner_up] = 10.0 - 1.0
    c[rows[:2], runner_up[:2]] = 10.0 + 0.3
    decisive = compare_logits(c, a2)
    assert decisive.decisive_disagreement_rate == pytest.approx(0.02) and decisive.worst_disagreement_gap > DECISIVE_GAP
    ok, why = decisive.verdict(torch.bfloat16)
    assert decisive.cosine > COSINE_FLOOR[torch.bfloat16] and not ok and "rank another token" in why


def test_non_finite_logits_and_shape_mismatches_are_refused():
    a = _logits()
    b = a.clone()
    b[3, 7] = float("nan")
    assert not compare_logits(b, a).verdict(torch.bfloat16)[0]
    with pytest.raises(ValueError, match="shapes differ"):
        compare_logits(a[:, :10], a)
    one = compare_logits(a[0], a[0])                      # a single row is a [1, vocab] comparison
    assert one.positions == 1 and "[same]" in report("row", one, torch.float32)
    assert isinstance(one, Agreement)


def test_the_first_divergent_layer_is_found_not_the_last():
    g = torch.Generator().manual_seed(3)
    a = [torch.randn(12, 32, generator=g) for _ in range(8)]
    b = [x.clone() for x in a]
    assert first_divergence(a, b) is None
    for layer in range(5, 8):                            # an error in layer 5 spoils every layer after it
        b[layer] = b[layer] + torch.randn(12, 32, generator=g)
    found = first_divergence(b, a)
    assert found is not None and found.layer == 5 and found.cosine < 0.9999
    with pytest.raises(ValueError):
        first_divergence(a[:3], a)
    c = [x.clone() for x in a]
    c[2] = c[2][:, :16]
    assert first_divergence(c, a).layer == 2              # a shape that differs is a divergence


def test_the_seeded_prompt_is_reproducible_and_inside_the_vocabulary():
    a, b = seeded_prompt(256, 100, 0), seeded_prompt(256, 100, 0)
    assert a == b and a != seeded_prompt(256, 100, 1) and min(a) >= 1 and max(a) < 256
    assert max(seeded_prompt(128256, 2000, 0)) < 30000


# ------------------------------------------------------------------ negative controls on the plain implementation
def _rms_inputs():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(8, 96, generator=g)
    x[2] *= 1e-4                                          # a nearly silent row: only there does eps matter
    x[5] *= 30.0
    x[6, -1] = 25.0                                       # a row whose last column carries most of its energy
    w = 1.0 + 0.1 * torch.randn(96, generator=g)
    return x, w


BROKEN_NORMS = {
    "missing_eps": lambda x, w, eps: x * torch.rsqrt((x * x).mean(-1, keepdim=True)) * w,
    "mean_over_the_wrong_axis": lambda x, w, eps: x * torch.rsqrt((x * x).mean(0, keepdim=True) + eps) * w,
    "dropped_last_column": lambda x, w, eps: x * torch.rsqrt((x[:, :-1] ** 2).sum(-1, keepdim=True) / x.shape[-1] + eps) * w,
    "half_a_percent_scale": lambda x, w, eps: 1.005 * plain.rms_norm(x, w, eps),
    "weight_before_the_normalisation": lambda x, w, eps: plain.rms_norm(x * w, torch.ones_like(w), eps),
    "sqrt_instead_of_rsqrt": lambda x, w, eps: x * torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w,
    "a_nan": lambda x, w, eps: plain.rms_norm(x, w, eps).index_put((torch.tensor([1]), torch.tensor([1])), torch.tensor(float("nan"))),
    "no_weight": lambda x, w, eps: plain.rms_norm(x, torch.ones_like(w), eps),
}


@pytest.mark.parametrize("name", sorted(BROKEN_NORMS))
def test_every_broken_norm_is_rejected(name):
    x, w = _rms_inputs()
    eps = 1e-5
    want = plain.rms_norm(x.double(), w.double(), eps)
    ok, _ = suite_compare(plain.rms_norm(x, w, eps), want, "float32")
    assert ok, "the comparison must accept the norm itself"
    ok, msg = suite_compare(BROKEN_NORMS[name](x, w, eps), want, "float32")
    assert not ok, f"{name} went through: {msg}"
    if name != "half_a_percent_scale":                    # half a percent is the size of bfloat16's own rounding
        ok, msg = suite_compare(BROKEN_NORMS[name](x, w, eps), want, "bfloat16")
        assert not ok, f"{name} went through at the bfloat16 tolerance: {msg}"


_attention = plain.causal_attention          # the controls below replace the module's attribute


def _off_by_one_mask(q, k, v, scale, window=None):
    n = q.shape[0]
    out = torch.empty_like(q)
    # query i also sees key i + 1
    group = q.shape[1] // k.shape[1]
    i, j = torch.arange(n).unsqueeze(1), torch.arange(n).unsqueeze(0)
    allowed = j <= i + 1
    for h in range(q.shape[1]):
        scores = (q[:, h] @ k[:, h // group].T) * scale
        out[:, h] = torch.softmax(scores.masked_fill(~allowed, float("-inf")), -1) @ v[:, h // group]
    return out


def _wrong_head_mapping(q, k, v, scale, window=None):
    nkv = k.shape[1]
    order = torch.tensor([h % nkv for h in range(q.shape[1])])     # head h reads key head h % nkv, not h // group
    return torch.stack([_attention(q[:, h:h + 1], k[:, order[h]:order[h] + 1], v[:, order[h]:order[h] + 1], scale, window)[:, 0]
                     for h in range(q.shape[1])], dim=1)


def _interleaved_rotation(x):
    out = torch.empty_like(x)
    out[..., 0::2] = -x[..., 1::2]
    out[..., 1::2] = x[..., 0::2]
    return out


MODEL_CONTROLS = {
    "off_by_one_mask": ("causal_attention", _off_by_one_mask),
    "wrong_gqa_head_mapping": ("causal_attention", _wrong_head_mapping),
    "interleaved_instead_of_half_rotation": ("rotate_half", _interleaved_rotation),
    "no_position_encoding": ("apply_rope", lambda x, cos, sin: x),
    "gelu_instead_of_silu": ("swiglu", lambda x, gate, up, down: (torch.nn.functional.gelu(x @ gate.T) * (x @ up.T)) @ down.T),
}


@pytest.mark.parametrize("name", sorted(MODEL_CONTROLS))
@pytest.mark.parametrize("tiny", ["A", "B"])
def test_a_broken_model_is_rejected_by_both_comparisons(monkeypatch, name, tiny):
    cfg = TINY[tiny]
    if name == "wrong_gqa_head_mapping" and cfg["num_key_value_heads"] == 1:
        pytest.skip("with one key head every mapping is the same")
    state = seeded_state(cfg, 21, std=0.2)              # large weights, so that attention is far from uniform
    tokens = seeded_tokens(40, cfg["vocab_size"], 5)
    want = plain.forward(cfg, state, tokens, torch.float64)
    assert suite_compare(plain.forward(cfg, state, tokens, torch.float32), want, "float32")[0]
    good_states: list = []
    plain.forward(cfg, state, tokens, torch.float64, good_states)
    attr, broken = MODEL_CONTROLS[name]
    monkeypatch.setattr(plain, attr, broken)
    bad_states: list = []
    got = plain.forward(cfg, state, tokens, torch.float64, bad_states)
    ok, msg = suite_compare(got, want, "bfloat16")
    assert not ok, f"{name} went through the suite's comparison: {msg}"
    ok, why = compare_logits(got, want).verdict(torch.bfloat16)
    assert not ok, f"{name} went through the equivalence verdict: {why}"
    assert first_divergence(bad_states, good_states).layer == 0, "the fault is in every layer, so the first one shows it"
