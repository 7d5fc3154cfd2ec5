"""A toy architecture defined in this test — never a model of anyone's — is
registered, built and stepped without any change to the package: a mixer with
state of its own (a running mean over the tokens seen so far) in one layer, a
windowed attention mixer in another, and a schedule that runs one layer twice.
It is replayed whole, in portions and mixed with other requests, and compared
with a plain composition of the same formulas."""

import pytest
import torch

import plain_llama as plain
import trace_modes as modes
from helpers import compare_logits, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu

TOY = {"architectures": ["ToyRunningMeanLM"], "hidden_size": 48, "vocab_size": 97, "intermediate_size": 80, "num_heads": 3,
       "num_kv_heads": 1, "head_dim": 16, "window": 9, "eps": 2e-5, "theta": 1000.0, "max_positions": 128}


def register_toy():
    from dataclasses import dataclass

    from stride_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
                                    register_architecture)
    from stride_b200.parts import Mixer, StateRequest, TensorDecl, register_part

    class RunningMeanMixer(Mixer):
        """delta_t = W * mean(x_0 .. x_t); the sum so far is per-request state."""
        graph_safe = False          # it walks the host's list of the step's requests

        def declare(self):
            h = self.spec.hidden
            return {self.spec.prefix + "mix.weight": TensorDecl((h, h))}

        def bind(self, weights):
            self.w = weights[self.spec.prefix + "mix.weight"]

        def state_request(self):
            return StateRequest((self.spec.hidden,), torch.float32)

        def forward(self, x, ctx, cache):
            out = self.rt.buffer("toy_mixer_out", x.shape[0], self.spec.hidden)
            for _request, row, n, position, slot in ctx.host_items:
                if position == 0:
                    cache.state[slot].zero_()
                sums = torch.cumsum(x[row: row + n].float(), 0) + cache.state[slot]
                cache.state[slot].copy_(sums[-1])
                counts = torch.arange(position + 1, position + n + 1, device=x.device, dtype=torch.float32).unsqueeze(1)
                out[row: row + n] = ((sums / counts).to(x.dtype).float() @ self.w.float().t()).to(x.dtype)
            return out

    @dataclass(frozen=True)
    class ToyConfig:
        d: tuple

        @classmethod
        def from_dict(cls, d):
            return cls(tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in d.items())))

        def to_dict(self):
            return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.d}

        def to_model_spec(self):
            c = self.to_dict()
            h = c["hidden_size"]
            norm = lambda p: NormSpec("rmsnorm", h, c["eps"], p)
            ffn = lambda p: FeedForwardSpec("swiglu", hidden=h, intermediate=c["intermediate_size"], prefix=p)
            attention = MixerSpec("attention", hidden=h, num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"],
                                  head_dim=c["head_dim"], scale=c["head_dim"] ** -0.5, window=c["window"],
                                  position=PositionSpec("rope", head_dim=c["head_dim"], theta=c["theta"],
                                                        max_positions=c["max_positions"]), prefix="toy.layers.0.self_attn.")
            mean = MixerSpec("toy_running_mean", hidden=h, prefix="toy.layers.1.")
            layers = (LayerSpec("pre_norm", attention, ffn("toy.layers.0.mlp."), norm("toy.layers.0.input_layernorm."),
                                norm("toy.layers.0.post_attention_layernorm.")),
                      LayerSpec("pre_norm", mean, ffn("toy.layers.1.mlp."), norm("toy.layers.1.n1."), norm("toy.layers.1.n2.")))
            # layer 0 runs twice, each run with a cache slot of its own
            schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2))
            return ModelSpec("ToyRunningMeanLM", h, c["vocab_size"], layers, schedule, norm("toy.norm."), "toy.embed.weight",
                             "toy.head.weight", c["max_positions"])

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_architecture("ToyRunningMeanLM", ToyConfig)


def toy_state(seed):
    g = torch.Generator().manual_seed(seed)
    c, h, i = TOY, TOY["hidden_size"], TOY["intermediate_size"]
    q, kv = c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]
    m = lambda r, k: torch.randn(r, k, generator=g) * 0.1
    v = lambda: 1 + 0.1 * torch.randn(h, generator=g)
    s = {"toy.embed.weight": m(c["vocab_size"], h), "toy.head.weight": m(c["vocab_size"], h), "toy.norm.weight": v(),
         "toy.layers.0.self_attn.q_proj.weight": m(q, h), "toy.layers.0.self_attn.k_proj.weight": m(kv, h),
         "toy.layers.0.self_attn.v_proj.weight": m(kv, h), "toy.layers.0.self_attn.o_proj.weight": m(h, q),
         "toy.layers.0.input_layernorm.weight": v(), "toy.layers.0.post_attention_layernorm.weight": v(),
         "toy.layers.1.mix.weight": m(h, h), "toy.layers.1.n1.weight": v(), "toy.layers.1.n2.weight": v()}
    for l in (0, 1):
        s.update({f"toy.layers.{l}.mlp.gate_proj.weight": m(i, h), f"toy.layers.{l}.mlp.up_proj.weight": m(i, h),
                  f"toy.layers.{l}.mlp.down_proj.weight": m(h, i)})
    return s


def plain_toy(state, tokens):
    w = {k: t.double() for k, t in state.items()}
    c = TOY
    cfg = {"num_attention_heads": c["num_heads"], "num_key_value_heads": c["num_kv_heads"], "head_dim": c["head_dim"],
           "hidden_size": c["hidden_size"]}
    cos, sin = plain.rope_tables(c["head_dim"], torch.arange(len(tokens)), c["theta"], None)
    x = w["toy.embed.weight"][torch.tensor(tokens)]

    def ffn(x, l, norm_name):
        h = plain.rms_norm(x, w[norm_name], c["eps"])
        return x + plain.swiglu(h, w[f"toy.layers.{l}.mlp.gate_proj.weight"], w[f"toy.layers.{l}.mlp.up_proj.weight"],
                                w[f"toy.layers.{l}.mlp.down_proj.weight"])

    def attention_layer(x):
        h = plain.rms_norm(x, w["toy.layers.0.input_layernorm.weight"], c["eps"])
        x = x + plain.attention_block(h, w, "toy.layers.0", cfg, cos.double(), sin.double(), c["window"])
        return ffn(x, 0, "toy.layers.0.post_attention_layernorm.weight")

    def mean_layer(x):
        h = plain.rms_norm(x, w["toy.layers.1.n1.weight"], c["eps"])
        mean = torch.cumsum(h, 0) / torch.arange(1, len(tokens) + 1, dtype=torch.float64).unsqueeze(1)
        x = x + mean @ w["toy.layers.1.mix.weight"].T
        return ffn(x, 1, "toy.layers.1.n2.weight")

    x = attention_layer(mean_layer(attention_layer(x)))
    return plain.rms_norm(x, w["toy.norm.weight"], c["eps"]) @ w["toy.head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_architecture_with_a_stateful_mixer_runs_through_the_engine(tmp_models, dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    register_toy()
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    state = toy_state(5)
    folder = write_model_dir(str(tmp_models / f"toy_{dtype}"), TOY, state, stored)
    state = {k: v.to(stored) for k, v in state.items()}
    requests = {r: seeded_tokens(n, TOY["vocab_size"], 900 + i) for i, (r, n) in enumerate({"a": 60, "b": 23, "c": 41, "d": 9}.items())}
    want = {r: plain_toy(state, t) for r, t in requests.items()}
    tol = "float32" if dtype == "float32" else "bfloat16"
    for name, steps in (("whole", modes.whole(requests)), ("portions", modes.changing_portions(requests)),
                        ("mixed", modes.mixed(requests, live_limit=3, seed=4))):
        session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=8)
        assert len(session.device_cache.groups) == 1 and session.device_cache.groups[0].window == TOY["window"]
        assert session.device_cache.groups[0].slots == (0, 2) and list(session.device_cache.states) == [1]
        assert not session.runner.cuda_graphs, "a part that reads the host's view of a step must not be graph-replayed"
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, (rid, pos) in enumerate(rows[s["step"]]):
                ok, msg = compare_logits(out[r:r + 1], want[rid][pos:pos + 1], tol)
                assert ok, f"{name}: request {rid!r} position {pos}: {msg}"
        stats = session.cache.stats()
        assert stats["live"] == 0 and session.cache.free_slots == session.cache.slot_capacity
        if name == "whole":
            assert stats["capacity"] * 8 >= 64, "sanity"
