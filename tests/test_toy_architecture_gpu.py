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
        """delta_t = W * mean(x_0 .. x_t); the sum so far is per-request state. Everything it needs of the step it
        takes from the step's arrays on the device (which sequence a token belongs to, where a sequence starts, its
        state slot), so a step that holds it can be captured in a graph and replayed. The framework hands out the
        slot and clears it when a request starts."""

        def declare(self):
            h = self.spec.hidden
            return {self.spec.prefix + "mix.weight": TensorDecl((h, h))}

        def bind(self, weights):
            self.w = weights[self.spec.prefix + "mix.weight"]

        def state_request(self):
            return StateRequest((self.spec.hidden,), torch.float32)

        def forward(self, x, ctx, cache):
            n = x.shape[0]
            seq = ctx.seq_of_token[:n].long()                   # -1: a padded row
            live = (seq >= 0).unsqueeze(1)
            seq = seq.clamp(min=0)
            start, count, slot = ctx.q_start.long(), ctx.q_len.long(), ctx.state_slot.long()
            running = torch.cumsum(torch.where(live, x.double(), 0.0), 0)                   # over the flat batch
            before = torch.where((start > 0).unsqueeze(1), running[(start - 1).clamp(min=0)], 0.0)      # [sequences, h]
            within = running - before[seq]                      # sum over the sequence's tokens of this step so far
            sums = within + cache.state[slot[seq]].double()
            mean = (sums / (ctx.positions[:n] + 1).double().unsqueeze(1)).to(x.dtype)
            # the state grows by the sum of the step's tokens; padded sequences (count 0) add nothing, whatever slot they name
            last = (start + count - 1).clamp(min=0)
            cache.state.index_add_(0, slot, torch.where((count > 0).unsqueeze(1), within[last], 0.0).float())
            out = self.rt.buffer("toy_mixer_out", n, self.spec.hidden)
            out.copy_((mean.float() @ self.w.float().t()).to(x.dtype))
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
    replays = 0
    for name, steps in (("whole", modes.whole(requests)), ("portions", modes.changing_portions(requests)),
                        ("tail", modes.tail_one_by_one(requests, tail=12)), ("mixed", modes.mixed(requests, live_limit=3, seed=4))):
        session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=8)
        assert len(session.device_cache.groups) == 1 and session.device_cache.groups[0].window == TOY["window"]
        assert session.device_cache.groups[0].slots == (0, 2) and list(session.device_cache.states) == [1]
        assert session.runner.cuda_graphs, "a mixer with state that reads the step from the device can be graph-replayed"
        for state in session.device_cache.states.values():      # whatever a slot held before: a new request starts at zero
            state.fill_(float("nan"))
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, (rid, pos) in enumerate(rows[s["step"]]):
                ok, msg = compare_logits(out[r:r + 1], want[rid][pos:pos + 1], tol)
                assert ok, f"{name}: request {rid!r} position {pos}: {msg}"
        stats = session.cache.stats()
        assert stats["live"] == 0 and session.cache.free_slots == session.cache.slot_capacity
        replays += session.runner.graph_replays
        if name == "whole":
            assert stats["capacity"] * 8 >= 64, "sanity"
        if name == "tail":
            assert session.runner.graph_replays >= 40, "the single-token steps did not go through captured graphs"
    assert replays > 0


# --------------------------------------------------------------------------------------------------------------
# A second toy: every kind of part that a layer is made of comes from this file — a norm that centres its input,
# a position encoding that adds a learned vector per position to queries and keys, a feed-forward that routes each
# token to one of three small experts, and an arrangement that feeds mixer and feed-forward from one norm in
# parallel. Only the attention mixer, the cache and the step function are the package's.
ROUTED = {"architectures": ["ToyRoutedLM"], "hidden_size": 40, "vocab_size": 83, "expert_width": 24, "experts": 3, "num_heads": 2,
          "num_kv_heads": 2, "head_dim": 16, "eps": 1e-4, "max_positions": 96, "layers": 2}


def register_routed_toy():
    from dataclasses import dataclass

    from stride_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
                                    register_architecture)
    from stride_b200.csrc import ops
    from stride_b200.parts import FeedForward, Layer, Norm, PositionEncoding, TensorDecl, build_part, register_part

    class CentredNorm(Norm):
        """y = (x - mean) * rsqrt(var + eps) * weight + bias, in float32."""

        def declare(self):
            w = self.spec.width
            return {self.spec.prefix + "weight": TensorDecl((w,), "vector"), self.spec.prefix + "bias": TensorDecl((w,), "vector")}

        def bind(self, weights):
            self.weight, self.bias = weights[self.spec.prefix + "weight"], weights[self.spec.prefix + "bias"]

        def apply(self, residual, pending, out, rows=None):
            x = residual if rows is None else residual[rows.long()]
            if pending is not None:
                x = x + (pending if rows is None else pending[rows.long()]).float()
                if rows is None:
                    residual.copy_(x)
            mean = x.mean(-1, keepdim=True)
            var = ((x - mean) ** 2).mean(-1, keepdim=True)
            out.copy_(((x - mean) * torch.rsqrt(var + self.spec.eps) * self.weight.float() + self.bias.float()).to(out.dtype))

    class LearnedOffset(PositionEncoding):
        """q and k of every head get table[position] added; keys and values are then stored as they are."""

        def declare(self):
            return {"toy.position.weight": TensorDecl((self.spec.max_positions, self.spec.head_dim))}

        def bind(self, weights):
            self.table = weights["toy.position.weight"]
            self._dummy = torch.zeros(8, dtype=torch.float32, device=self.table.device)

        def encode_and_store(self, qkv, bias, ctx, cache, num_heads, num_kv_heads, head_dim):
            tokens = qkv.shape[0]
            offsets = self.table[ctx.positions[:tokens].long()].float()                     # [tokens, head_dim]
            rotated = (num_heads + num_kv_heads) * head_dim
            view = qkv[:, :rotated].view(tokens, num_heads + num_kv_heads, head_dim)
            view.copy_((view.float() + offsets.unsqueeze(1)).to(qkv.dtype))
            ops.rope_kv_write(qkv, bias, ctx.positions[:tokens], ctx.slot_mapping[cache.group][:tokens] if cache.writes else None,
                              self._dummy, self._dummy, cache.k_pages, cache.v_pages, num_heads, num_kv_heads, head_dim,
                              cache.page_size, rotate=False)

    class TopOneExperts(FeedForward):
        """Router logits in float32; the token goes to the expert with the largest one and its output is weighted
        with that expert's softmax probability. Expert: down(relu(up(x)))."""

        def _names(self, e):
            p = self.spec.prefix
            return p + f"experts.{e}.up.weight", p + f"experts.{e}.down.weight"

        def declare(self):
            params = dict(self.spec.params)
            h, w, n = self.spec.hidden, params["expert_width"], params["experts"]
            d = {self.spec.prefix + "router.weight": TensorDecl((n, h))}
            for e in range(n):
                up, down = self._names(e)
                d[up], d[down] = TensorDecl((w, h)), TensorDecl((h, w))
            return d

        def bind(self, weights):
            n = dict(self.spec.params)["experts"]
            self.router = weights[self.spec.prefix + "router.weight"]
            self.up = torch.stack([weights[self._names(e)[0]] for e in range(n)])
            self.down = torch.stack([weights[self._names(e)[1]] for e in range(n)])

        def forward(self, x, ctx):
            logits = x.float() @ self.router.float().t()                                    # router in float32
            prob = torch.softmax(logits, -1)
            choice = logits.argmax(-1)
            hidden = torch.relu(torch.einsum("th,ewh->tew", x.float(), self.up.float())).to(x.dtype).float()
            outs = torch.einsum("tew,ehw->teh", hidden, self.down.float())                  # every expert, then one is picked
            picked = outs[torch.arange(x.shape[0], device=x.device), choice] * prob.gather(1, choice[:, None])
            out = self.rt.buffer("toy_routed_out", x.shape[0], self.spec.hidden)
            out.copy_(picked.to(out.dtype))
            return out

    class ParallelLayer(Layer):
        """x += mixer(n(x)) + ffn(n(x)) with one norm."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.norm = build_part("norm", spec.mixer_norm, runtime)
            self.mixer = build_part("mixer", spec.mixer, runtime)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime)

        def parts(self):
            return (self.norm, self.mixer, self.feed_forward)

        def declare(self):
            d = {}
            for p in self.parts():
                d.update(p.declare())
            return d

        def bind(self, weights):
            for p in self.parts():
                p.bind(weights)

        def forward(self, stream, ctx, cache):
            h = stream.normed(self.norm)
            stream.add(self.mixer.forward(h, ctx, cache))
            stream.add(self.feed_forward.forward(h, ctx))

    @dataclass(frozen=True)
    class RoutedConfig:
        d: tuple

        @classmethod
        def from_dict(cls, d):
            return cls(tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in d.items())))

        def to_dict(self):
            return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.d}

        def to_model_spec(self):
            c = self.to_dict()
            h = c["hidden_size"]
            norm = lambda p: NormSpec("toy_centred", h, c["eps"], p)
            position = PositionSpec("toy_learned_offset", head_dim=c["head_dim"], max_positions=c["max_positions"])
            layers = []
            for l in range(c["layers"]):
                mixer = MixerSpec("attention", hidden=h, num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"],
                                  head_dim=c["head_dim"], scale=c["head_dim"] ** -0.5, position=position,
                                  prefix=f"toy.layers.{l}.self_attn.")
                ffn = FeedForwardSpec("toy_top_one", hidden=h, prefix=f"toy.layers.{l}.moe.",
                                      params=(("expert_width", c["expert_width"]), ("experts", c["experts"])))
                layers.append(LayerSpec("toy_parallel", mixer, ffn, norm(f"toy.layers.{l}.norm."), norm(f"toy.layers.{l}.norm.")))
            schedule = tuple(ScheduleEntry(l, l) for l in range(c["layers"]))
            return ModelSpec("ToyRoutedLM", h, c["vocab_size"], tuple(layers), schedule, norm("toy.norm."), "toy.embed.weight",
                             "toy.head.weight", c["max_positions"])

    register_part("norm", "toy_centred", CentredNorm)
    register_part("position", "toy_learned_offset", LearnedOffset)
    register_part("feed_forward", "toy_top_one", TopOneExperts)
    register_part("layer", "toy_parallel", ParallelLayer)
    register_architecture("ToyRoutedLM", RoutedConfig)


def routed_state(seed):
    g = torch.Generator().manual_seed(seed)
    c, h = ROUTED, ROUTED["hidden_size"]
    q = c["num_heads"] * c["head_dim"]
    m = lambda r, k, s=0.15: torch.randn(r, k, generator=g) * s
    v = lambda: 1 + 0.1 * torch.randn(h, generator=g)
    b = lambda: 0.1 * torch.randn(h, generator=g)
    s = {"toy.embed.weight": m(c["vocab_size"], h, 1.0), "toy.head.weight": m(c["vocab_size"], h), "toy.norm.weight": v(),
         "toy.norm.bias": b(), "toy.position.weight": m(c["max_positions"], c["head_dim"], 0.5)}
    for l in range(c["layers"]):
        p = f"toy.layers.{l}."
        s.update({p + "self_attn.q_proj.weight": m(q, h), p + "self_attn.k_proj.weight": m(q, h), p + "self_attn.v_proj.weight": m(q, h),
                  p + "self_attn.o_proj.weight": m(h, q), p + "norm.weight": v(), p + "norm.bias": b(),
                  p + "moe.router.weight": m(c["experts"], h, 1.0)})
        for e in range(c["experts"]):
            s[p + f"moe.experts.{e}.up.weight"] = m(c["expert_width"], h)
            s[p + f"moe.experts.{e}.down.weight"] = m(h, c["expert_width"])
    return s


def plain_routed(state, tokens):
    """The same formulas, whole sequence, float64; returns the logits and the smallest gap between the two largest
    router logits (a position whose gap is tiny may be routed differently by a path that rounds differently)."""
    w = {k: t.double() for k, t in state.items()}
    c = ROUTED
    n, hd, nh = len(tokens), c["head_dim"], c["num_heads"]
    x = w["toy.embed.weight"][torch.tensor(tokens)]
    offsets = w["toy.position.weight"][:n]
    gap = float("inf")

    def norm(x, p):
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return (x - mean) * torch.rsqrt(var + c["eps"]) * w[p + "weight"] + w[p + "bias"]

    for l in range(c["layers"]):
        p = f"toy.layers.{l}."
        h = norm(x, p + "norm.")
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(n, nh, hd) + offsets[:, None]
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(n, nh, hd) + offsets[:, None]
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(n, nh, hd)
        scores = torch.einsum("qhd,khd->hqk", q, k) * hd ** -0.5
        scores = scores.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
        attn = torch.einsum("hqk,khd->qhd", torch.softmax(scores, -1), v).reshape(n, nh * hd) @ w[p + "self_attn.o_proj.weight"].T
        logits = h @ w[p + "moe.router.weight"].T
        top = logits.topk(2, -1).values
        gap = min(gap, float((top[:, 0] - top[:, 1]).min()))
        prob, choice = torch.softmax(logits, -1), logits.argmax(-1)
        moe = torch.zeros_like(x)
        for t in range(n):
            e = int(choice[t])
            moe[t] = (torch.relu(h[t] @ w[p + f"moe.experts.{e}.up.weight"].T) @ w[p + f"moe.experts.{e}.down.weight"].T) * prob[t, e]
        x = x + attn + moe
    return norm(x, "toy.norm.") @ w["toy.head.weight"].T, gap


def test_a_toy_architecture_of_foreign_parts_runs_through_the_engine(tmp_models):
    """float32 only: a routed feed-forward is discontinuous, and in bfloat16 a token near a tie may take another
    expert than in float64 without anything being wrong."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    register_routed_toy()
    state = routed_state(7)
    folder = write_model_dir(str(tmp_models / "toy_routed"), ROUTED, state, torch.float32)
    requests = {r: seeded_tokens(n, ROUTED["vocab_size"], 700 + i) for i, (r, n) in enumerate({"a": 50, "b": 17, "c": 33}.items())}
    want = {}
    for r, t in requests.items():
        want[r], gap = plain_routed(state, t)
        assert gap > 1e-4, "the test's weights put a token on a routing tie; change the seed"
    for name, steps in (("whole", modes.whole(requests)), ("portions", modes.changing_portions(requests)),
                        ("mixed", modes.mixed(requests, live_limit=3, seed=5))):
        session = TraceSession(folder, "float32", max_tokens=modes.peak_tokens(steps), block_size=8)
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, (rid, pos) in enumerate(rows[s["step"]]):
                ok, msg = compare_logits(out[r:r + 1], want[rid][pos:pos + 1], "float32")
                assert ok, f"{name}: request {rid!r} position {pos}: {msg}"
        assert session.cache.stats()["live"] == 0


# --------------------------------------------------------------------------------------------------------------
# A third toy: the two ends of the model and what the mixer keeps in pages come from this file. The embedding is a
# table lookup times sqrt(width); the head adds a bias and caps the logits with a tanh; the mixer keeps ONE vector of
# 24 numbers per token in the pages (not keys and values), attends over those vectors and projects the weighted
# vector back. Norms, feed-forward, arrangement, cache manager and step function are the package's.
LATENT = {"architectures": ["ToyLatentLM"], "hidden_size": 56, "vocab_size": 101, "intermediate_size": 72, "latent": 24, "eps": 1e-5,
          "cap": 4.0, "max_positions": 160, "layers": 2}


def register_latent_toy():
    from dataclasses import dataclass

    from stride_b200.config import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, ScheduleEntry,
                                    register_architecture)
    from stride_b200.parts import CacheRequest, Embedding, Head, Mixer, TensorDecl, register_part

    class ScaledLookup(Embedding):
        def declare(self):
            return {self.spec.name: TensorDecl((self.spec.vocab, self.spec.hidden))}

        def bind(self, weights):
            self.weight = weights[self.spec.name]

        def forward(self, ctx, out):
            n = out.shape[0]
            live = (ctx.seq_of_token[:n] >= 0).unsqueeze(1)
            rows = self.weight[ctx.token_ids[:n].long()].float() * dict(self.spec.params)["multiplier"]
            out.copy_(torch.where(live, rows, 0.0))

    class CappedHead(Head):
        def declare(self):
            return {self.spec.name: TensorDecl((self.spec.vocab, self.spec.hidden)),
                    self.spec.name.replace("weight", "bias"): TensorDecl((self.spec.vocab,), "vector")}

        def bind(self, weights, tied=None):
            self.weight, self.bias = weights[self.spec.name], weights[self.spec.name.replace("weight", "bias")]

        def forward(self, x, out):
            cap = dict(self.spec.params)["cap"]
            out.copy_(cap * torch.tanh((x.float() @ self.weight.float().t() + self.bias) / cap))

    class LatentMixer(Mixer):
        """c_t = Wc x_t is what a token leaves in the cache; delta_t = Wo sum_j softmax_j(q_t . c_j / sqrt(r)) c_j over j <= t."""
        graph_safe = False          # it walks the host's list of the step's requests

        def declare(self):
            h, r, p = self.spec.hidden, dict(self.spec.params)["latent"], self.spec.prefix
            return {p + "c.weight": TensorDecl((r, h)), p + "q.weight": TensorDecl((r, h)), p + "o.weight": TensorDecl((h, r))}

        def bind(self, weights):
            p = self.spec.prefix
            self.wc, self.wq, self.wo = weights[p + "c.weight"], weights[p + "q.weight"], weights[p + "o.weight"]

        def cache_request(self):
            return CacheRequest(tensors=(("latent", 1, dict(self.spec.params)["latent"]),))

        def forward(self, x, ctx, cache):
            r = self.wc.shape[0]
            pages = cache.tensors["latent"]                             # [num_pages, 1, page_size, r]
            flat = pages.view(-1, r)                                    # one head: row = page * page_size + offset
            n = x.shape[0]
            c = (x.float() @ self.wc.float().t()).to(x.dtype)
            q = (x.float() @ self.wq.float().t()).to(x.dtype).float()
            slots = ctx.slot_mapping[cache.group][:n].long()
            live = slots >= 0
            flat[slots[live]] = c[live]
            out = self.rt.buffer("toy_latent_out", n, self.spec.hidden)
            out.zero_()
            table = ctx.block_table[cache.group]
            for index, (_request, row, count, position, _slot) in enumerate(ctx.host_items):
                end = position + count
                at = torch.arange(end, device=x.device)
                kept = flat[table[index, at // cache.page_size].long() * cache.page_size + at % cache.page_size].float()      # [end, r]
                scores = q[row:row + count] @ kept.t() * r ** -0.5
                mask = at.unsqueeze(0) > (position + torch.arange(count, device=x.device)).unsqueeze(1)
                weights = torch.softmax(scores.masked_fill(mask, float("-inf")), -1)
                out[row:row + count] = ((weights @ kept).to(x.dtype).float() @ self.wo.float().t()).to(x.dtype)
            return out

    @dataclass(frozen=True)
    class LatentConfig:
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
            layers = tuple(LayerSpec("pre_norm", MixerSpec("toy_latent", hidden=h, prefix=f"toy.layers.{l}.mix.", params=(("latent", c["latent"]),)),
                                     FeedForwardSpec("swiglu", hidden=h, intermediate=c["intermediate_size"], prefix=f"toy.layers.{l}.mlp."),
                                     norm(f"toy.layers.{l}.n1."), norm(f"toy.layers.{l}.n2.")) for l in range(c["layers"]))
            return ModelSpec("ToyLatentLM", h, c["vocab_size"], layers, tuple(ScheduleEntry(l, l) for l in range(c["layers"])),
                             norm("toy.norm."), "toy.embed.weight", "toy.head.weight", c["max_positions"],
                             embedding=EmbeddingSpec("toy_scaled_lookup", c["vocab_size"], h, "toy.embed.weight", (("multiplier", h ** 0.5),)),
                             head=HeadSpec("toy_capped", c["vocab_size"], h, "toy.head.weight", (("cap", c["cap"]),)))

    register_part("embedding", "toy_scaled_lookup", ScaledLookup)
    register_part("head", "toy_capped", CappedHead)
    register_part("mixer", "toy_latent", LatentMixer)
    register_architecture("ToyLatentLM", LatentConfig)


def latent_state(seed):
    g = torch.Generator().manual_seed(seed)
    c, h, r, i = LATENT, LATENT["hidden_size"], LATENT["latent"], LATENT["intermediate_size"]
    m = lambda rows, cols, s=0.15: torch.randn(rows, cols, generator=g) * s
    v = lambda: 1 + 0.1 * torch.randn(h, generator=g)
    s = {"toy.embed.weight": m(c["vocab_size"], h, 0.1), "toy.head.weight": m(c["vocab_size"], h, 0.3),
         "toy.head.bias": torch.randn(c["vocab_size"], generator=g) * 0.5, "toy.norm.weight": v()}
    for l in range(c["layers"]):
        p = f"toy.layers.{l}."
        s.update({p + "mix.c.weight": m(r, h, 0.12), p + "mix.q.weight": m(r, h, 0.12), p + "mix.o.weight": m(h, r), p + "n1.weight": v(),
                  p + "n2.weight": v(), p + "mlp.gate_proj.weight": m(i, h), p + "mlp.up_proj.weight": m(i, h),
                  p + "mlp.down_proj.weight": m(h, i)})
    return s


def plain_latent(state, tokens):
    w = {k: t.double() for k, t in state.items()}
    c = LATENT
    n, r = len(tokens), c["latent"]
    x = w["toy.embed.weight"][torch.tensor(tokens)] * c["hidden_size"] ** 0.5
    for l in range(c["layers"]):
        p = f"toy.layers.{l}."
        h = plain.rms_norm(x, w[p + "n1.weight"], c["eps"])
        kept, q = h @ w[p + "mix.c.weight"].T, h @ w[p + "mix.q.weight"].T
        scores = (q @ kept.T * r ** -0.5).masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
        x = x + torch.softmax(scores, -1) @ kept @ w[p + "mix.o.weight"].T
        h = plain.rms_norm(x, w[p + "n2.weight"], c["eps"])
        x = x + plain.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    logits = plain.rms_norm(x, w["toy.norm.weight"], c["eps"]) @ w["toy.head.weight"].T + w["toy.head.bias"]
    return c["cap"] * torch.tanh(logits / c["cap"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_with_its_own_ends_and_one_cached_vector_per_token_runs_through_the_engine(tmp_models, dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    register_latent_toy()
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    state = latent_state(9)
    folder = write_model_dir(str(tmp_models / f"toy_latent_{dtype}"), LATENT, state, stored)
    state = {k: v.to(stored) for k, v in state.items()}
    requests = {r: seeded_tokens(n, LATENT["vocab_size"], 800 + i) for i, (r, n) in enumerate({"a": 70, "b": 19, "c": 44, "d": 5}.items())}
    want = {r: plain_latent(state, t) for r, t in requests.items()}
    for name, steps in (("whole", modes.whole(requests)), ("tail", modes.tail_one_by_one(requests, tail=10)),
                        ("portions", modes.changing_portions(requests)), ("mixed", modes.mixed(requests, live_limit=3, seed=6))):
        session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=8)
        group = session.device_cache.groups[0]
        assert group.layout == (("latent", 1, LATENT["latent"]),) and group.slots == (0, 1)
        assert [tuple(t.shape[2:]) for t in session.device_cache.pages] == [(1, 8, LATENT["latent"])], "one vector per token is kept"
        for pages in session.device_cache.pages:
            pages.fill_(float("nan"))
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, (rid, pos) in enumerate(rows[s["step"]]):
                ok, msg = compare_logits(out[r:r + 1], want[rid][pos:pos + 1], dtype)
                assert ok, f"{name}: request {rid!r} position {pos}: {msg}"
        assert session.cache.stats()["live"] == 0
