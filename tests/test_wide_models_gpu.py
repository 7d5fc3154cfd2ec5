"""Whole models of width 1024 with weights of standard deviation 0.05: the shapes at which bfloat16 logits drift
furthest from float64 (scores of a few units, so that the rounding of the normed activations and of the queries
and keys passes through the softmax's exponent).

float32 is held to the same bound as everywhere. For bfloat16 the cosine floor of the tiny configurations (0.9995,
taken from a comparison of two bfloat16 runs, python/stride_worker/diagnose/equivalence.py:40-44) does not apply to
a comparison with float64 at these shapes: the reference's own bfloat16 model falls below it on the same input.
The bound here is therefore a relative one, measured in the same run: the engine may not be further from float64
than the plain implementation is when it computes in bfloat16 (every operation rounded, as the reference's
``F.linear`` and attention in bfloat16 are), neither in the mean relative error of a row nor in its worst cosine;
and where the reference's package is at hand (``baseline/_ref``), its mean relative error may not exceed that of
the reference's own bfloat16 model on the same rows either.
"""

import os
import sys

import pytest
import torch

import plain_llama as plain
import trace_modes as modes
from helpers import compare_logits, seeded_state, seeded_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu", "hidden_size": 1024}
LLAMA3 = {"rope_type": "llama3", "low_freq_factor": 1.0}
WIDE = {
    "one_key_head_tied": (dict(head_dim=64, num_key_value_heads=1, num_attention_heads=4, intermediate_size=512, vocab_size=32000,
                               num_hidden_layers=3, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=4096,
                               tie_word_embeddings=True), 102, [7, 33, 65, 150, 300]),
    "no_groups_eps_3e-4": (dict(head_dim=64, num_key_value_heads=4, num_attention_heads=4, intermediate_size=384, vocab_size=1000,
                                num_hidden_layers=2, rms_norm_eps=3e-4, rope_theta=1234.5, max_position_embeddings=1024,
                                rope_scaling=dict(LLAMA3, factor=2.0, high_freq_factor=2.0, original_max_position_embeddings=256),
                                tie_word_embeddings=False), 106, [300, 2, 257]),
    "sixteen_heads_bias": (dict(head_dim=64, num_key_value_heads=4, num_attention_heads=16, intermediate_size=512, vocab_size=1000,
                                num_hidden_layers=2, rms_norm_eps=1e-5, rope_theta=1234.5, max_position_embeddings=4096,
                                rope_scaling=dict(LLAMA3, factor=8.0, high_freq_factor=4.0, original_max_position_embeddings=32),
                                tie_word_embeddings=False, attention_bias=True), 130, [150, 2, 300, 300]),
    "one_head_of_128": (dict(head_dim=128, num_key_value_heads=1, num_attention_heads=1, intermediate_size=384, vocab_size=32000,
                             num_hidden_layers=1, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=1024,
                             rope_scaling=dict(LLAMA3, factor=8.0, high_freq_factor=4.0, original_max_position_embeddings=64),
                             tie_word_embeddings=True), 136, [65, 65, 100, 257, 33, 150]),
}


def distance(got: torch.Tensor, want: torch.Tensor):
    """(mean over rows of |got - want| / |want|, worst cosine of a row), in float64."""
    a, b = got.double(), want.double()
    rel = (a - b).norm(dim=-1) / b.norm(dim=-1)
    return float(rel.mean()), float(torch.nn.functional.cosine_similarity(a, b, dim=-1).min())


def reference_bfloat16(cfg, state, requests, keep):
    """Logits of the reference's own model in bfloat16 at the kept places, or None when its package is not here."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        from stride_worker.cache import PagedKVCache
        from stride_worker.model import StrideModel
        from stride_worker.protocol import SequenceWork
    except ImportError:
        return None
    finally:
        sys.path.pop(0)
    model = StrideModel(dict(cfg), {k: v.cuda() for k, v in state.items()}, torch.device("cuda"), torch.bfloat16)
    got = {}
    for rid, tokens in requests.items():
        pages = (len(tokens) + 15) // 16
        cache = PagedKVCache(model.cache_spec(pages + 1, 16))
        at = 0
        for end in sorted(p + 1 for p in keep[rid]):
            _, logits, _ = model.forward([SequenceWork(seq=0, tokens=tokens[at:end], position=at, blocks=list(range(pages)),
                                                       needs_logits=True)], cache)
            got[(rid, end - 1)] = logits[0].float().cpu()
            at = end
    return got


@pytest.mark.parametrize("name", sorted(WIDE))
def test_width_1024_float32_and_bfloat16_against_float64(tmp_models, name):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    from helpers import write_model_dir
    sizes, seed, lengths = WIDE[name]
    cfg = dict(BASE, **sizes)
    state = seeded_state(cfg, seed, std=0.05)
    if cfg.get("attention_bias"):
        g = torch.Generator().manual_seed(99)
        nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        for i in range(cfg["num_hidden_layers"]):
            for proj, rows in (("q", nq * hd), ("k", nkv * hd), ("v", nkv * hd)):
                state[f"model.layers.{i}.self_attn.{proj}_proj.bias"] = torch.randn(rows, generator=g) * 0.1
    requests = {chr(97 + i): seeded_tokens(n, cfg["vocab_size"], 10 * seed + i) for i, n in enumerate(lengths)}
    keep = {rid: set(range(0, len(t), 11)) | set(range(max(0, len(t) - 34), len(t))) for rid, t in requests.items()}
    cuttings = {"whole": modes.whole(requests), "tail": modes.tail_one_by_one(requests), "portions": modes.changing_portions(requests),
                "mixed": modes.mixed(requests, live_limit=4, seed=seed)}
    for dtype, stored in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        rounded = {k: v.to(stored) for k, v in state.items()}                # bfloat16: the rounded weights are the model
        on_gpu = {k: v.cuda() for k, v in rounded.items()}
        want, yardstick = {}, {}
        for rid, tokens in requests.items():
            places = sorted(keep[rid])
            exact = plain.forward(cfg, on_gpu, tokens, torch.float64)[places].cpu()
            want.update({(rid, p): exact[i] for i, p in enumerate(places)})
            if dtype == "bfloat16":
                rough = plain.forward(cfg, on_gpu, tokens, torch.bfloat16)[places].float().cpu()
                yardstick.update({(rid, p): rough[i] for i, p in enumerate(places)})
        folder = write_model_dir(str(tmp_models / f"wide_{name}_{dtype}"), cfg, state, stored)
        if dtype == "bfloat16":
            keys = sorted(want)
            exact = torch.stack([want[k] for k in keys])
            plain_mean, plain_cos = distance(torch.stack([yardstick[k] for k in keys]), exact)
            ref = reference_bfloat16(cfg, rounded, requests, keep)
        for mode, steps in cuttings.items():
            steps = modes.restrict_wants([dict(s, entries=[dict(e) for e in s["entries"]]) for s in steps], keep)
            session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=16)
            rows, got = modes.expected_rows(steps), {}
            for s in steps:
                out = session.run_step(s)
                for r, key in enumerate(rows[s["step"]]):
                    got[key] = out[r].clone()
            keys = sorted(got)
            assert len(keys) >= 30
            a, b = torch.stack([got[k] for k in keys]), torch.stack([want[k] for k in keys])
            if dtype == "float32":
                ok, msg = compare_logits(a, b, dtype)
                assert ok, f"{name} float32 {mode}: {msg}"
                continue
            mean, cos = distance(a, b)
            sub_mean, sub_cos = distance(torch.stack([yardstick[k] for k in keys]), b)
            where = f"{name} bfloat16 {mode}: engine mean relative error {mean:.4f}, worst cosine {cos:.6f}"
            assert torch.isfinite(a).all(), where
            assert mean <= sub_mean and cos >= sub_cos, f"{where}; the plain implementation in bfloat16: {sub_mean:.4f}, {sub_cos:.6f}"
            assert mean <= plain_mean, f"{where}; the plain implementation in bfloat16 over all kept rows: {plain_mean:.4f}"
            if ref is not None:
                r_mean, r_cos = distance(torch.stack([ref[k] for k in keys]), b)
                # the mean over the rows only: the worst of a hundred rows is one draw, and two bfloat16 computations
                # that round at different places trade it back and forth (0.999115 here against 0.999131 there)
                assert mean <= r_mean, f"{where}; the reference's model in bfloat16: {r_mean:.4f}, {r_cos:.6f}"
            print(f"{where} | plain bf16 {sub_mean:.4f} {sub_cos:.6f} | reference bf16 "
                  + (f"{r_mean:.4f} {r_cos:.6f}" if ref is not None else "not at hand"))
