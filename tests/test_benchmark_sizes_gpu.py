"""Whole-model logits at the layer sizes that the benchmark runs: hidden 4096, 32 query and 8 key heads of 128,
inner width 14336, a vocabulary of 128256 and llama3 frequency scaling, with two layers instead of 32 so that it
fits a test. The composed bfloat16 path of a decode step (norms folded into the products, rotation and cache write
in the QKV epilogue, split decode attention, gated tcgen05 product, tcgen05 head) and the prefill path are replayed
whole, with the last tokens one by one, in portions of changing size and mixed in a small pool, in float32 and in
bfloat16, and compared with the plain implementation in float64. The reference compares whole-model logits on the
real shape in the same way (python/stride_worker/diagnose/prefill.py:21-107, diagnose/equivalence.py:100-149).

The weights are drawn on the GPU (1.5 G numbers) and the plain implementation runs there in float64, which is the
one place where it leaves the CPU; nothing is written to disk.
"""

import pytest
import torch

import plain_llama as plain
import trace_modes as modes
from helpers import compare_logits, geometry, seeded_tokens

pytestmark = pytest.mark.gpu

SIZES = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 2048,
    "hidden_act": "silu",
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
LENGTHS = {"a": 600, "b": 333, "c": 47, "d": 130}
STORED = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def drawn_on_the_gpu(cfg: dict, seed: int, std: float = 0.02, norm_jitter: float = 0.1) -> dict:
    """float32 weights by checkpoint name, N(0, std), norm weights 1 + N(0, norm_jitter), from one CUDA generator."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    nq, nkv, hd = geometry(cfg)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]

    def mat(rows, cols):
        return torch.randn(rows, cols, generator=g, device="cuda") * std

    def norm():
        return 1.0 + torch.randn(H, generator=g, device="cuda") * norm_jitter

    state = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        state[f"{p}.input_layernorm.weight"] = norm()
        state[f"{p}.self_attn.q_proj.weight"] = mat(nq * hd, H)
        state[f"{p}.self_attn.k_proj.weight"] = mat(nkv * hd, H)
        state[f"{p}.self_attn.v_proj.weight"] = mat(nkv * hd, H)
        state[f"{p}.self_attn.o_proj.weight"] = mat(H, nq * hd)
        state[f"{p}.post_attention_layernorm.weight"] = norm()
        state[f"{p}.mlp.gate_proj.weight"] = mat(I, H)
        state[f"{p}.mlp.up_proj.weight"] = mat(I, H)
        state[f"{p}.mlp.down_proj.weight"] = mat(H, I)
    state["model.norm.weight"] = norm()
    state["lm_head.weight"] = mat(V, H)
    return state


class Case:
    """The model in one element type with what the plain implementation says, and the replays made so far."""

    def __init__(self, dtype: str, requests: dict, keep: dict):
        from stride_b200.config import config_from_dict
        from stride_b200.engine.loading import build_model
        from stride_b200.weights import DictSource
        self.dtype, self.requests, self.keep = dtype, requests, keep
        state = {k: v.to(STORED[dtype]) for k, v in drawn_on_the_gpu(SIZES, 8).items()}      # bfloat16: the rounded weights are the model
        exact = {k: v.double() for k, v in state.items()}
        self.want = {}
        for rid, tokens in requests.items():
            logits = plain.forward(SIZES, exact, tokens, torch.float64)
            self.want.update({(rid, p): logits[p].cpu() for p in keep[rid]})
        del exact, logits
        self.config = config_from_dict(dict(SIZES))
        self.model = build_model(self.config, DictSource(state), dtype, "cuda", token_capacity=2048, row_capacity=256)
        self.replays = {}

    def replay(self, mode: str) -> dict:
        if mode not in self.replays:
            from stride_b200.engine.trace import TraceSession
            requests = self.requests
            steps = {"whole": lambda: modes.whole(requests), "tail": lambda: modes.tail_one_by_one(requests),
                     "portions": lambda: modes.changing_portions(requests), "mixed": lambda: modes.mixed(requests, live_limit=4, seed=5),
                     "mixed_3_live": lambda: modes.mixed(requests, live_limit=3, seed=2, decode_tail=20)}[mode]()
            steps = modes.restrict_wants(steps, self.keep)
            session = TraceSession(None, self.dtype, max_tokens=modes.peak_tokens(steps), block_size=16, model=self.model,
                                   config=self.config)
            rows, got = modes.expected_rows(steps), {}
            for s in steps:
                out = session.run_step(s)
                for r, key in enumerate(rows[s["step"]]):
                    got[key] = out[r].clone()
            stats = session.cache.stats()
            assert stats["live"] == 0 and stats["free"] == stats["capacity"], "pages were lost"
            self.replays[mode] = got
        return self.replays[mode]


@pytest.fixture(scope="module")
def cases():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    requests = {rid: seeded_tokens(n, SIZES["vocab_size"], 900 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
    # logits are wanted at the first places, at every 29th and at the last 34 of each request (a row is half a megabyte)
    keep = {rid: set(range(0, len(t), 29)) | {1, 2} & set(range(len(t))) | set(range(max(0, len(t) - 34), len(t)))
            for rid, t in requests.items()}
    made = {}

    def get(dtype):
        if dtype not in made:
            made[dtype] = Case(dtype, requests, keep)
        return made[dtype]

    yield get
    made.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_gives_the_plain_logits_at_the_benchmark_sizes(cases, dtype, mode):
    case = cases(dtype)
    got = case.replay(mode)
    # a cutting returns the places it wants among those kept: all of them when whole, the last 33 of each request
    # when they are decoded one by one, first and last places of portions otherwise
    assert set(got) <= set(case.want) and len(got) >= (len(case.want) if mode == "whole" else 60), len(got)
    keys = sorted(got)
    ok, msg = compare_logits(torch.stack([got[k] for k in keys]), torch.stack([case.want[k] for k in keys]), dtype)
    assert ok, f"{dtype} {mode}: {msg}"


def test_float32_is_bitwise_the_same_under_every_cutting_at_the_benchmark_sizes(cases):
    case = cases("float32")
    base = case.replay("whole")
    for mode in ("tail", "portions", "mixed", "mixed_3_live"):
        for key, row in case.replay(mode).items():
            assert torch.equal(row, base[key]), f"{mode}: request {key[0]!r} position {key[1]} differs from the whole run"


@pytest.mark.parametrize("live", [20, 33, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_decoding_together_at_the_benchmark_sizes(cases, dtype, live):
    """Decode-only steps of 20, 33 and 64 rows (the graph buckets 32 and 64; above 16 rows the library products
    and the norm, rotation and SiLU kernels as launches of their own) after prompts of different lengths."""
    from stride_b200.engine.trace import TraceSession
    case = cases(dtype)
    requests = {f"r{i}": seeded_tokens(9 + (i * 7) % 61, SIZES["vocab_size"], 2000 + i) for i in range(live)}
    exact = {k: v.double() for k, v in case.model.named_tensors().items()}
    steps = modes.decoding_together(requests, decode_steps=8)
    session = TraceSession(None, dtype, max_tokens=modes.peak_tokens(steps), block_size=16, max_requests=live, model=case.model,
                           config=case.config)
    rows, got = modes.expected_rows(steps), {}
    for s in steps:
        out = session.run_step(s)
        for r, key in enumerate(rows[s["step"]]):
            got[key] = out[r].clone()
    assert session.runner.graph_replays >= 7, "the decode steps did not go through captured graphs"
    want = {}
    for rid, tokens in requests.items():
        logits = plain.forward(SIZES, exact, tokens, torch.float64)
        want.update({(rid, p): logits[p].cpu() for (r, p) in got if r == rid})
    keys = sorted(got)
    assert len(keys) == live * 9
    ok, msg = compare_logits(torch.stack([got[k] for k in keys]), torch.stack([want[k] for k in keys]), dtype)
    assert ok, f"{live} requests decoding together, {dtype}: {msg}"
