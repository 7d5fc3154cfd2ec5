"""Whole models at sizes that the fast kernels do not take, so that every fallback is walked: a width that is no
multiple of 8, head sizes 80 and 144, a projection bias, a tied head, a prime vocabulary. Each is replayed with the
last tokens one by one and mixed with other requests, in float32 and bfloat16, against the plain implementation."""

import pytest
import torch

import plain_llama as plain
import trace_modes as modes
from helpers import compare_logits, seeded_state, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False, "max_position_embeddings": 512, "hidden_act": "silu"}
ODD = {
    "width_100_head_80": dict(num_hidden_layers=2, hidden_size=100, num_attention_heads=5, num_key_value_heads=1, head_dim=80,
                              intermediate_size=120, vocab_size=333),
    "bias_and_group_2": dict(num_hidden_layers=2, hidden_size=136, num_attention_heads=6, num_key_value_heads=3, head_dim=64,
                             intermediate_size=200, vocab_size=1001, attention_bias=True),
    "head_144_tied": dict(num_hidden_layers=1, hidden_size=256, num_attention_heads=3, num_key_value_heads=3, head_dim=144,
                          intermediate_size=448, vocab_size=4099, tie_word_embeddings=True),
}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_sizes_take_the_fallbacks_and_stay_right(tmp_models, name, dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    cfg = dict(BASE)
    cfg.update(ODD[name])
    state = seeded_state(cfg, 11, std=0.05)
    if cfg.get("attention_bias"):
        g = torch.Generator().manual_seed(99)
        nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        for i in range(cfg["num_hidden_layers"]):
            for proj, rows in (("q", nq * hd), ("k", nkv * hd), ("v", nkv * hd)):
                state[f"model.layers.{i}.self_attn.{proj}_proj.bias"] = torch.randn(rows, generator=g) * 0.1
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_model_dir(str(tmp_models / f"odd_{name}_{dtype}"), cfg, state, stored)
    state = {k: v.to(stored) for k, v in state.items()}
    requests = {"a": seeded_tokens(150, cfg["vocab_size"], 1), "b": seeded_tokens(37, cfg["vocab_size"], 2),
                "c": seeded_tokens(90, cfg["vocab_size"], 3)}
    want = {r: plain.forward(cfg, state, t, torch.float64) for r, t in requests.items()}
    for mode, steps in (("tail", modes.tail_one_by_one(requests)), ("mixed", modes.mixed(requests, live_limit=3, seed=7))):
        session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=16)
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, (rid, pos) in enumerate(rows[s["step"]]):
                ok, msg = compare_logits(out[r:r + 1], want[rid][pos:pos + 1], dtype)
                assert ok, f"{name} {dtype} {mode}: request {rid!r} position {pos}: {msg}"
