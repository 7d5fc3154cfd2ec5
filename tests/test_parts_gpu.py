"""Each part alone on the GPU against the plain implementation: norm through the
residual stream, rotary tables, the feed-forward, and the attention mixer with a
window and biases, run in portions through the cache manager."""

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu
DTYPES = [("float32", torch.float32, 3e-6), ("bfloat16", torch.bfloat16, 2e-2)]


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def runtime_for(dtype, tokens=64, rows=16):
    from stride_b200.parts import Runtime
    return Runtime("cuda", dtype, tokens, rows)


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= tol * scale, f"max abs error {err:.3e} against scale {scale:.3e}"


def step_context(cache, items, groups=1, device="cuda"):
    """items: [(request key, tokens, position, want)] -> StepContext on the device."""
    from stride_b200.cache import runtime
    from stride_b200.engine.context import make_context
    batch = runtime().StepBatch(cache)
    host = []
    row = 0
    for key, tokens, position, want in items:
        batch.add(key, tokens, position, want)
        host.append((key, row, len(tokens), position, cache.state_slot(key)))
        row += len(tokens)
    arr, layout = batch.pack(groups, max(batch.num_tokens, 1), max(batch.num_seqs, 1), max(batch.num_rows, 1),
                             max(batch.max_pages, 1))
    dev = torch.from_numpy(arr).to(device)
    return make_context(dev, layout, batch.num_tokens, batch.num_seqs, batch.num_rows, max_q_len=batch.max_q_len,
                        max_ctx=batch.max_ctx, decode_only=batch.decode_only, host_items=host)


@pytest.mark.parametrize("name,dtype,tol", DTYPES)
def test_norm_through_the_residual_stream(gpu, name, dtype, tol):
    from stride_b200.config import NormSpec
    from stride_b200.parts import ResidualStream, build_part
    rt = runtime_for(dtype)
    g = torch.Generator().manual_seed(1)
    norm = build_part("norm", NormSpec("rmsnorm", 88, 3e-5, "n."), rt)
    assert list(norm.declare()) == ["n.weight"] and norm.declare()["n.weight"].role == "vector"
    w = 1 + 0.3 * torch.randn(88, generator=g)
    norm.bind({"n.weight": w.cuda()})
    x0 = torch.randn(10, 88, generator=g)
    d1 = torch.randn(10, 88, generator=g).to(dtype)
    d2 = torch.randn(10, 88, generator=g).to(dtype)
    stream = ResidualStream(rt, 10, 88)
    stream.residual.copy_(x0)
    stream.add(d1.cuda())
    out1 = stream.normed(norm).clone()
    close(out1, plain.rms_norm(x0.double() + d1.double(), w.double(), 3e-5), tol)
    stream.add(d2.cuda())
    stream.add(d1.cuda())          # two pending sums: the first is applied at once
    rows = torch.tensor([9, 2], dtype=torch.int32, device="cuda")
    total = x0.double() + 2 * d1.double() + d2.double()
    close(stream.normed(norm, rows=rows), plain.rms_norm(total[[9, 2]], w.double(), 3e-5), tol)
    close(stream.materialize(), total, 3e-6)


def test_rotary_tables_follow_the_reference_formula(gpu):
    from stride_b200.config import PositionSpec, RopeScaling
    from stride_b200.parts import build_part
    rt = runtime_for(torch.float32)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    spec = PositionSpec("rope", head_dim=32, theta=500000.0, max_positions=300, scaling=RopeScaling(**scaling))
    cos, sin = build_part("position", spec, rt).tables()
    want_cos, want_sin = plain.rope_tables(32, torch.arange(300), 500000.0, scaling)
    assert torch.equal(cos.cpu(), want_cos[:, :16]) and torch.equal(sin.cpu(), want_sin[:, :16])
    plain_spec = PositionSpec("rope", head_dim=32, theta=500000.0, max_positions=300, scaling=None)
    assert not torch.equal(build_part("position", plain_spec, rt).tables()[0].cpu(), cos.cpu())


@pytest.mark.parametrize("name,dtype,tol", DTYPES)
def test_feed_forward_alone(gpu, name, dtype, tol):
    from stride_b200.config import FeedForwardSpec
    from stride_b200.parts import build_part
    rt = runtime_for(dtype)
    g = torch.Generator().manual_seed(2)
    ffn = build_part("feed_forward", FeedForwardSpec("swiglu", hidden=88, intermediate=136, prefix="f."), rt)
    w = {"f.gate_proj.weight": torch.randn(136, 88, generator=g) * 0.2, "f.up_proj.weight": torch.randn(136, 88, generator=g) * 0.2,
         "f.down_proj.weight": torch.randn(88, 136, generator=g) * 0.2}
    assert {k: v.shape for k, v in ffn.declare().items()} == {k: tuple(v.shape) for k, v in w.items()}
    w = {k: v.to(dtype) for k, v in w.items()}
    ffn.bind({k: v.cuda() for k, v in w.items()})
    assert all(torch.equal(ffn.named_tensors()[k].cpu(), v) for k, v in w.items())
    x = torch.randn(13, 88, generator=g).to(dtype)
    got = ffn.forward(x.cuda(), None)
    close(got, plain.swiglu(x.double(), *(w[k].double() for k in w)), tol)
    with pytest.raises(ValueError, match="gelu"):
        build_part("feed_forward", FeedForwardSpec("swiglu", hidden=8, intermediate=8, activation="gelu"), rt)
    with pytest.raises(ValueError, match="no feed_forward of kind"):
        build_part("feed_forward", FeedForwardSpec("experts", hidden=8), rt)


@pytest.mark.parametrize("name,dtype,tol", DTYPES)
@pytest.mark.parametrize("window,bias", [(None, False), (11, True)])
def test_attention_mixer_alone_in_portions(gpu, name, dtype, tol, window, bias):
    """Two requests run in portions and single tokens through the mixer; pages of
    the windowed case are given back while the request runs."""
    from stride_b200.cache import CacheManager, DeviceCache
    from stride_b200.config import MixerSpec, PositionSpec
    from stride_b200.parts import build_part
    rt = runtime_for(dtype)
    g = torch.Generator().manual_seed(3)
    H, nq, nkv, hd, page = 72, 6, 2, 32, 8
    spec = MixerSpec("attention", hidden=H, num_heads=nq, num_kv_heads=nkv, head_dim=hd, scale=hd ** -0.5, window=window,
                     bias=bias, position=PositionSpec("rope", head_dim=hd, theta=10000.0, max_positions=256), prefix="a.self_attn.")
    mixer = build_part("mixer", spec, rt)
    w = {"a.self_attn.q_proj.weight": torch.randn(nq * hd, H, generator=g) * 0.2,
         "a.self_attn.k_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.2,
         "a.self_attn.v_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.2,
         "a.self_attn.o_proj.weight": torch.randn(H, nq * hd, generator=g) * 0.2}
    if bias:
        for k, n in (("q", nq * hd), ("k", nkv * hd), ("v", nkv * hd)):
            w[f"a.self_attn.{k}_proj.bias"] = torch.randn(n, generator=g) * 0.1
    assert set(mixer.declare()) == set(w)
    w = {k: (v.to(dtype) if v.dim() == 2 else v) for k, v in w.items()}
    mixer.bind({k: v.cuda() for k, v in w.items()})
    assert mixer.cache_request().window == window

    class OneMixerModel:                      # the least a DeviceCache needs to know
        schedule = [type("E", (), {"layer": 0, "cache": 0, "writes_cache": True})()]
        def cache_requests(self):
            return [(mixer.cache_request(), None)]
    model = OneMixerModel()
    device_cache = DeviceCache(model, page, 16 if window is None else 9, 4, dtype, "cuda")
    for p in device_cache.pages:
        p.fill_(float("nan"))
    cache = CacheManager(page, device_cache.group_configs(), 4, False)
    lengths = {1: 70, 2: 37}
    xs = {k: torch.randn(n, H, generator=g).to(dtype) for k, n in lengths.items()}
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": H}
    want = {}
    for k, x in xs.items():
        cos, sin = plain.rope_tables(hd, torch.arange(len(x)), 10000.0, None)
        want[k] = plain.attention_block(x.double(), {n: t.double() for n, t in w.items()}, "a", cfg, cos.double(), sin.double(), window)
    held = {1: 0, 2: 0}
    plan = [[(1, 24), (2, 5)], [(1, 1), (2, 16)], [(1, 2)], [(1, 40), (2, 1)], [(2, 15), (1, 1)], [(1, 2)]]
    cache.open(1), cache.open(2)
    for step in plan:
        items = []
        for key, n in step:
            assert cache.ensure(key, held[key] + n, 0)
            items.append((key, list(range(n)), held[key], []))
        ctx = step_context(cache, items)
        x = torch.cat([xs[key][held[key]: held[key] + n] for key, n in step]).cuda()
        out = mixer.forward(x, ctx, model.caches[0])
        row = 0
        for key, n in step:
            close(out[row: row + n], want[key][held[key]: held[key] + n], tol)
            row += n
            held[key] += n
            cache.trim(key, held[key])
        cache.check_invariants()
    assert held == lengths
    if window:
        assert cache.table(1, 0).count(-1) >= 6, "the window never gave a page back"
        assert cache.stats()["live"] <= 6
