"""Seeded random configurations of the architecture, replayed under every cutting against the plain implementation:
head sizes in steps of 16 up to 256, any number of heads and groups, widths and vocabularies that are no power of
two, with and without llama3 frequency scaling, tied and untied heads, projection biases. Half of them have the sizes
that the tensor-core kernels take (head size 64 or 128, group up to 8), the other half walks the fallbacks.

float32: the usual bound against float64, and bitwise the same logits under every cutting. bfloat16: finite, and no
further from float64 (mean relative error of a row) than the plain implementation computed in bfloat16; the absolute
cosine floor of the tiny configurations does not hold for every random shape at weights of standard deviation 0.05
(see tests/test_wide_models_gpu.py).
"""

import random

import pytest
import torch

import plain_llama as plain
import trace_modes as modes
from helpers import compare_logits, seeded_biases, seeded_state, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu"}
COUNT = 10


def configuration(index: int):
    rng = random.Random(7000 + index)
    c = dict(BASE)
    if index % 2 == 0:
        nkv, group = rng.choice([1, 2, 4]), rng.choice([1, 2, 4, 8])
        c.update(head_dim=rng.choice([64, 128]), num_key_value_heads=nkv, num_attention_heads=nkv * group,
                 hidden_size=rng.choice([128, 256, 384, 512, 1024]), intermediate_size=rng.choice([256, 384, 512, 1024, 1408]),
                 vocab_size=rng.choice([512, 1000, 4096, 32000]), num_hidden_layers=rng.choice([1, 2, 3]))
    else:
        nkv, group = rng.randint(1, 4), rng.choice([1, 1, 2, 3, 5, 7, 16, 20])
        c.update(head_dim=16 * rng.randint(1, 16), num_key_value_heads=nkv, num_attention_heads=nkv * group,
                 hidden_size=rng.choice([36, 50, 77, 100, 136, 200, 264, 520]), intermediate_size=rng.choice([40, 99, 150, 272, 500]),
                 vocab_size=rng.choice([97, 333, 1001, 5003]), num_hidden_layers=rng.choice([1, 2, 4]))
    c["rms_norm_eps"] = rng.choice([1e-5, 1e-6, 3e-4])
    c["rope_theta"] = rng.choice([10000.0, 500000.0, 1234.5])
    c["max_position_embeddings"] = rng.choice([1024, 2048, 4096])
    if rng.random() < 0.5:
        c["rope_scaling"] = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]), "low_freq_factor": 1.0,
                             "high_freq_factor": rng.choice([2.0, 4.0]), "original_max_position_embeddings": rng.choice([32, 64, 256])}
    c["tie_word_embeddings"] = rng.random() < 0.4
    c["attention_bias"] = rng.random() < 0.3
    lengths = [rng.choice([1, 2, 7, 33, 64, 65, 100, 150, 257]) for _ in range(rng.randint(3, 5))]
    return c, lengths, rng.choice([8, 16, 16, 32])


def relative_error(got, want):
    a, b = got.double(), want.double()
    return float(((a - b).norm(dim=-1) / b.norm(dim=-1).clamp_min(1e-12)).mean())


@pytest.mark.parametrize("index", range(COUNT))
def test_a_random_configuration_under_every_cutting(tmp_models, index):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    cfg, lengths, page = configuration(index)
    state = seeded_state(cfg, 100 + index, std=0.05)
    if cfg["attention_bias"]:
        state.update(seeded_biases(cfg, 99))
    requests = {chr(97 + i): seeded_tokens(n, cfg["vocab_size"], 10 * index + i) for i, n in enumerate(lengths)}
    cuttings = {"whole": lambda: modes.whole(requests), "tail": lambda: modes.tail_one_by_one(requests),
                "portions": lambda: modes.changing_portions(requests), "mixed": lambda: modes.mixed(requests, live_limit=4, seed=index)}
    what = f"configuration {index} {dict((k, v) for k, v in cfg.items() if k not in BASE)}, page {page}"
    for dtype, stored in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        folder = write_model_dir(str(tmp_models / f"random_{index}_{dtype}"), cfg, state, stored)
        rounded = {k: v.to(stored) for k, v in state.items()}
        want = {r: plain.forward(cfg, rounded, t, torch.float64) for r, t in requests.items()}
        rough = {r: plain.forward(cfg, rounded, t, torch.bfloat16).float() for r, t in requests.items()} if dtype == "bfloat16" else None
        first = {}
        for mode, make in cuttings.items():
            steps = make()
            session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=page)
            rows, got = modes.expected_rows(steps), {}
            for s in steps:
                out = session.run_step(s)
                for r, key in enumerate(rows[s["step"]]):
                    got[key] = out[r].clone()
            keys = sorted(got)
            a = torch.stack([got[k] for k in keys])
            b = torch.stack([want[r][p] for r, p in keys])
            if dtype == "float32":
                ok, msg = compare_logits(a, b, dtype)
                assert ok, f"{what}, float32 {mode}: {msg}"
                for k in keys:
                    assert torch.equal(first.setdefault(k, got[k]), got[k]), \
                        f"{what}, float32 {mode}: request {k[0]!r} position {k[1]} differs from the first cutting that gave it"
            else:
                assert torch.isfinite(a).all(), f"{what}, bfloat16 {mode}: non-finite logits"
                mine, yardstick = relative_error(a, b), relative_error(torch.stack([rough[r][p] for r, p in keys]), b)
                assert mine <= yardstick, (f"{what}, bfloat16 {mode}: mean relative error {mine:.4f}; the plain implementation "
                                           f"in bfloat16 has {yardstick:.4f}")
            assert session.cache.stats()["live"] == 0
