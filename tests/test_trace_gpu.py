"""Trace replay on the GPU against the plain implementation: the same requests
whole, with the last tokens one by one, in portions of changing size, and mixed
with other requests in a pool so small that pages are used again; in float32 and
in bfloat16; in process and through bin/trace_run."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as plain
import trace_modes as modes
from helpers import PAGE_SIZE, TINY, compare_logits, read_model_dir, seeded_state, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"a": 70, "b": 33, "c": 161, "d": 17, "e": 2, "f": 64, "g": 230}


@pytest.fixture(scope="module", params=["A", "B", "C", "D"])
def case(request, tmp_models):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    name = request.param
    cfg = TINY[name]
    out = {"name": name, "cfg": cfg, "page": PAGE_SIZE[name], "dirs": {}, "want": {}}
    state = seeded_state(cfg, 40 + ord(name))
    out["requests"] = {rid: seeded_tokens(n, cfg["vocab_size"], 300 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
    for dtype, stored in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        d = write_model_dir(str(tmp_models / f"{name}_{dtype}"), cfg, state, stored)
        out["dirs"][dtype] = d
        _, stored_state = read_model_dir(d)     # bfloat16: the rounded weights are the model
        out["want"][dtype] = {rid: plain.forward(cfg, stored_state, t, torch.float64) for rid, t in out["requests"].items()}
    return out


def session_for(case, dtype, steps, graphs=True, slack_pages=0):
    from stride_b200.engine.trace import TraceSession
    return TraceSession(case["dirs"][dtype], dtype, max_tokens=modes.peak_tokens(steps) + slack_pages * case["page"],
                        block_size=case["page"], cuda_graphs=graphs)


def replay(session, steps):
    """(request, position) -> float32 logits row."""
    rows = modes.expected_rows(steps)
    got = {}
    for s in steps:
        out = session.run_step(s)
        wanted = rows[s["step"]]
        assert (out is None) == (not wanted)
        if wanted:
            assert out.shape[0] == len(wanted)
            for r, key in enumerate(wanted):
                got[key] = out[r].clone()
    return got


def check(got, want, dtype, what):
    keys = sorted(got)
    a = torch.stack([got[k] for k in keys])
    b = torch.stack([want[rid][pos] for rid, pos in keys])
    ok, msg = compare_logits(a, b, dtype)
    if not ok:
        bad = ((a.double() - b).abs().max(-1).values).argmax()
        msg += f"; worst at request {keys[int(bad)][0]!r} position {keys[int(bad)][1]}"
    assert ok, f"{what}: {msg}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_requests(case, dtype):
    steps = modes.whole(case["requests"])
    got = replay(session_for(case, dtype, steps), steps)
    assert len(got) == sum(LENGTHS.values())
    check(got, case["want"][dtype], dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["tail", "portions", "mixed"])
def test_cuttings_agree_with_the_plain_implementation(case, dtype, mode):
    requests = case["requests"]
    steps = {"tail": lambda: modes.tail_one_by_one(requests), "portions": lambda: modes.changing_portions(requests),
             "mixed": lambda: modes.mixed(requests, seed=5)}[mode]()
    session = session_for(case, dtype, steps)
    got = replay(session, steps)
    check(got, case["want"][dtype], dtype, mode)
    stats = session.cache.stats()
    assert stats["live"] == 0 and stats["free"] == stats["capacity"], "pages were lost"


def test_float32_logits_are_bitwise_the_same_under_every_cutting(case):
    requests = case["requests"]
    base_steps = modes.whole(requests)
    base = replay(session_for(case, "float32", base_steps), base_steps)
    for name, steps in (("tail", modes.tail_one_by_one(requests)), ("portions", modes.changing_portions(requests)),
                        ("mixed", modes.mixed(requests, seed=9)), ("mixed2", modes.mixed(requests, live_limit=3, seed=2))):
        got = replay(session_for(case, "float32", steps), steps)
        for key, row in got.items():
            assert torch.equal(row, base[key]), f"{name}: request {key[0]!r} position {key[1]} differs from the whole run"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_are_used_again_and_old_contents_do_not_leak(case, dtype):
    requests = case["requests"]
    steps = modes.mixed(requests, live_limit=2, seed=3)
    session = session_for(case, dtype, steps)
    pool = session.cache.stats()["capacity"]
    assert pool * case["page"] < sum(LENGTHS.values()), "the pool is large enough to avoid reuse; the test would show nothing"
    # poison the pool: stale contents of a reused page must never be read
    for pages in session.device_cache.pages:
        pages.fill_(float("nan"))
    got = replay(session, steps)
    check(got, case["want"][dtype], dtype, "reused pages")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(case, dtype):
    tokens = case["requests"]["c"]
    steps = [{"step": 0, "entries": [{"id": "c", "tokens": tokens[:3], "want": [0, 1, 2]}], "end": []}]
    for p in range(3, len(tokens)):
        steps.append({"step": p, "entries": [{"id": "c", "tokens": [tokens[p]], "want": [0]}], "end": []})
    steps[-1]["end"] = ["c"]
    for graphs in (True, False):
        session = session_for(case, dtype, steps, graphs=graphs)
        got = replay(session, steps)
        check(got, case["want"][dtype], dtype, f"decode one by one (graphs={graphs})")
        if graphs:
            assert session.runner.graph_replays > 100, "decode steps did not go through captured graphs"


def test_decoding_across_context_buckets(case, monkeypatch):
    """A decode graph is captured for a bound on the context; a request that grows past it moves to the graph
    of the next bound. With a small first bound the 161 tokens of request c cross two of them."""
    from stride_b200.engine.runner import ModelRunner
    monkeypatch.setattr(ModelRunner, "CONTEXT_BUCKET_BASE", 16)
    tokens = case["requests"]["c"]
    steps = [{"step": 0, "entries": [{"id": "c", "tokens": tokens[:3], "want": [0, 1, 2]}], "end": []}]
    for p in range(3, len(tokens)):
        steps.append({"step": p, "entries": [{"id": "c", "tokens": [tokens[p]], "want": [0]}], "end": []})
    steps[-1]["end"] = ["c"]
    session = session_for(case, "bfloat16", steps, graphs=True)
    got = replay(session, steps)
    check(got, case["want"]["bfloat16"], "bfloat16", "decode across context buckets")
    assert len({k[1] for k in session.runner._graphs if k[0] != "portion"}) >= 3, "the context never moved to another graph"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [20, 33, 64])
def test_many_requests_decoding_together(case, dtype, live):
    """Up to 64 requests live at once, all decoding in the same steps: the decode graphs for 32 and 64 rows, where
    the bfloat16 products go to the library and norm, rotation and SiLU run as kernels of their own."""
    from stride_b200.engine.trace import TraceSession
    vocab = case["cfg"]["vocab_size"]
    requests = {f"r{i}": seeded_tokens(9 + (i * 7) % 41, vocab, 3000 + i) for i in range(live)}
    _, state = read_model_dir(case["dirs"][dtype])
    want = {rid: plain.forward(case["cfg"], state, t, torch.float64) for rid, t in requests.items()}
    steps = modes.decoding_together(requests, decode_steps=8)
    session = TraceSession(case["dirs"][dtype], dtype, max_tokens=modes.peak_tokens(steps), block_size=case["page"], max_requests=live)
    got = replay(session, steps)
    assert len(got) == live * 9
    check(got, want, dtype, f"{live} requests decoding together")
    assert session.runner.graph_replays >= 7, "the decode steps did not go through captured graphs"
    assert max(session.runner.captured_buckets()) >= min(live, 64)


@pytest.mark.parametrize("live", [20, 33, 64, 100])
def test_many_requests_decoding_together_on_the_tokens_as_rows_products(case, live, monkeypatch):
    """The package's own tcgen05 products with fused epilogues for 17 to 128 tokens are off by default (the library
    product is as fast or faster); here they take every decode step of more than 16 tokens."""
    from stride_b200.csrc import ops
    from stride_b200.engine.trace import TraceSession
    monkeypatch.setattr(ops, "ROWS_GEMM_MAX_TOKENS", 128)
    taken = {}
    for name in ("linear_rows_qkv_rope", "linear_rows_add_norm", "linear_rows_gated"):
        def counted(*args, _f=getattr(ops, name), _name=name, **kwargs):
            done = _f(*args, **kwargs)
            taken[_name] = taken.get(_name, 0) + bool(done)
            return done
        monkeypatch.setattr(ops, name, counted)
    vocab = case["cfg"]["vocab_size"]
    requests = {f"r{i}": seeded_tokens(9 + (i * 7) % 41, vocab, 3000 + i) for i in range(live)}
    _, state = read_model_dir(case["dirs"]["bfloat16"])
    want = {rid: plain.forward(case["cfg"], state, t, torch.float64) for rid, t in requests.items()}
    steps = modes.decoding_together(requests, decode_steps=6)
    session = TraceSession(case["dirs"]["bfloat16"], "bfloat16", max_tokens=modes.peak_tokens(steps), block_size=case["page"], max_requests=live)
    got = replay(session, steps)
    check(got, want, "bfloat16", f"{live} requests decoding together on the tokens-as-rows products")
    if case["name"] == "D":       # its sizes are the kernels': all three must have run, with the norms folded into them
        assert all(taken.get(n, 0) > 0 for n in ("linear_rows_qkv_rope", "linear_rows_add_norm", "linear_rows_gated")), taken
    assert session.runner.graph_replays >= 5, "the decode steps did not go through captured graphs"


def test_an_unknown_token_or_too_few_pages_is_an_error_not_a_wrong_result(case):
    from stride_b200.engine.trace import TraceError, TraceSession
    s = TraceSession(case["dirs"]["float32"], "float32", max_tokens=64, block_size=case["page"])
    with pytest.raises(TraceError, match="vocabulary"):
        s.run_step({"step": 0, "entries": [{"id": "x", "tokens": [case["cfg"]["vocab_size"]], "want": [0]}], "end": []})
    with pytest.raises(TraceError, match="out of cache pages"):
        s.run_step({"step": 1, "entries": [{"id": "y", "tokens": [1] * 65, "want": [64]}], "end": []})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_run_program(case, dtype, tmp_path):
    requests = {k: case["requests"][k] for k in ("a", "b", "d", "e")}
    steps = modes.mixed(requests, live_limit=4, seed=11)
    out_dir = tmp_path / "logits"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", case["dirs"][dtype], "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(modes.peak_tokens(steps)),
                           "--block-size", str(case["page"])],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    rows = modes.expected_rows(steps)
    got = {}
    vocab = case["cfg"]["vocab_size"]
    for s in steps:
        path = out_dir / f"{s['step']}.f32"
        if not rows[s["step"]]:
            assert not path.exists()
            continue
        data = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
        assert data.shape[0] == len(rows[s["step"]])
        for r, key in enumerate(rows[s["step"]]):
            got[key] = torch.from_numpy(data[r].copy())
    check(got, case["want"][dtype], dtype, "bin/trace_run")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_trace_may_run_past_the_length_that_the_checkpoint_names(tmp_models, dtype):
    """The rotation is defined for every position; ``max_position_embeddings`` only sizes the table. A replay of
    300 given tokens through a model that names 256 positions gives the plain logits at every position."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.engine.trace import TraceSession
    cfg = TINY["A"]
    assert cfg["max_position_embeddings"] == 256
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_model_dir(str(tmp_models / f"past_the_end_{dtype}"), cfg, seeded_state(cfg, 91, std=0.05), stored)
    _, state = read_model_dir(folder)
    requests = {"long": seeded_tokens(300, cfg["vocab_size"], 17)}
    want = {"long": plain.forward(cfg, state, requests["long"], torch.float64)}
    for steps in (modes.whole(requests), modes.tail_one_by_one(requests, tail=60)):
        session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=16)
        assert session.model.spec.max_positions >= 300
        check(replay(session, steps), want, dtype, "past max_position_embeddings")
