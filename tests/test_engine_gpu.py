"""Generation through the Python entry point and the command line on the GPU,
against the plain implementation: greedy tokens, prefix-cache hits,
preempt-and-resume, stop rules, seeded temperature sampling."""

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as plain
from helpers import PAGE_SIZE, TINY, read_model_dir, seeded_state, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", params=["A", "B"])
def case(request, tmp_models):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    name = request.param
    cfg = TINY[name]
    state = seeded_state(cfg, 70 + ord(name), std=0.08)      # larger weights: decisive argmax gaps
    out = {"name": name, "cfg": cfg, "page": PAGE_SIZE[name], "dirs": {}, "state": {}}
    for dtype, stored in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        out["dirs"][dtype] = write_model_dir(str(tmp_models / f"gen_{name}_{dtype}"), cfg, state, stored)
        out["state"][dtype] = read_model_dir(out["dirs"][dtype])[1]
    lengths = [1, 7, 16, 33] if name == "A" else [3, 25, 41, 57, 72, 90]
    shared = seeded_tokens(24, cfg["vocab_size"], 500)
    out["prompts"] = [(shared[:min(24, n - 1)] + seeded_tokens(n, cfg["vocab_size"], 501 + i))[:n] if name == "B"
                      else seeded_tokens(n, cfg["vocab_size"], 501 + i) for i, n in enumerate(lengths)]
    out["new_tokens"] = 8 if name == "A" else 12
    return out


def engine_for(case, dtype, **options):
    from stride_b200 import Engine
    options.setdefault("block_size", case["page"])
    options.setdefault("num_blocks", 64)
    options.setdefault("max_model_len", case["cfg"]["max_position_embeddings"])
    options.setdefault("check_invariants", True)
    return Engine(case["dirs"][dtype], dtype=dtype, **options)


def assert_greedy(case, dtype, prompt, generated, what=""):
    """Teacher-forced check: every generated token is the plain argmax, or, in
    bfloat16, within rounding of it."""
    logits = plain.forward(case["cfg"], case["state"][dtype], list(prompt) + list(generated), torch.float64)
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        if dtype == "float32":
            assert tok == int(row.argmax()), f"{what}: token {i} is {tok}, the plain argmax is {int(row.argmax())}"
        else:
            gap = float(row.max() - row[tok])
            assert gap <= 0.03 * float(row.abs().max()), f"{what}: token {i} is {gap:.3g} below the plain maximum"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(case, dtype):
    from stride_b200 import SamplingParams
    engine = engine_for(case, dtype)
    n = case["new_tokens"]
    # two waves: pages are published when a request ends, so the second wave can find the shared prefix
    params = SamplingParams(temperature=0.0, max_tokens=n)
    outs = engine.generate(case["prompts"][:2], params) + engine.generate(case["prompts"][2:], params)
    for prompt, out in zip(case["prompts"], outs):
        assert out.finished and out.finish_reason == "length" and len(out.tokens) == n and out.prompt_len == len(prompt)
        assert_greedy(case, dtype, prompt, out.tokens, f"prompt of {len(prompt)}")
    if dtype == "float32":
        for prompt, out in zip(case["prompts"], outs):
            assert out.tokens == plain.greedy_generate(case["cfg"], case["state"][dtype], prompt, n, torch.float64)
    m = engine.metrics()
    assert m["finished"] == len(outs) and m["kv_blocks_live"] == 0 and m["graph_replays"] > 0
    last = engine.last_step          # the record of the last step: a decode of the requests still running
    assert last["decode_only"] and last["tokens"] == last["seqs"] == last["rows"] >= 1 and last["us"] > 0
    if case["name"] == "B":
        assert m["prefill_tokens_reused"] > 0, "the shared 24-token prefix was never found in the cache"


def test_small_budgets_small_pools_and_resume_give_the_same_tokens(case):
    """Portions of 5..16 tokens, a pool that cannot hold every request, so that
    requests are preempted and recomputed, with and without the prefix index."""
    from stride_b200 import SamplingParams
    n = case["new_tokens"] + 20
    want = [plain.greedy_generate(case["cfg"], case["state"]["float32"], p, n, torch.float64) for p in case["prompts"]]
    longest = max(len(p) for p in case["prompts"]) + n
    pages = -(-longest // case["page"]) + 3
    for prefix_caching in (True, False):
        engine = engine_for(case, "float32", num_blocks=pages, max_batch_tokens=16, max_batch_seqs=4, watermark=0.0,
                            prefix_caching=prefix_caching)
        outs = engine.generate(case["prompts"], SamplingParams(temperature=0.0, max_tokens=n))
        assert [o.tokens for o in outs] == want
        m = engine.metrics()
        assert m["preemptions"] > 0, "the pool was meant to be too small"
        assert m["kv_blocks_live"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_alone_is_prefilled_in_full_portions_from_a_graph(case, dtype):
    """One request whose prompt is several token budgets long: every portion but the last fills the budget and is
    replayed from the graph captured for such portions; the tokens are the plain ones."""
    from stride_b200 import SamplingParams
    prompt = seeded_tokens(3 * 16 + 5, case["cfg"]["vocab_size"], 777)
    engine = engine_for(case, dtype, max_batch_tokens=16, max_batch_seqs=4)
    out = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6))[0]
    assert_greedy(case, dtype, prompt, out.tokens, "full portions from a graph")
    assert ("portion", 0) in engine.runner._graphs, "no full portion went through the graph"
    replays = engine.runner.graph_replays
    again = engine.generate([prompt[:40] + prompt[:13]], SamplingParams(temperature=0.0, max_tokens=6))[0]       # other positions, same graph
    assert_greedy(case, dtype, prompt[:40] + prompt[:13], again.tokens, "full portions from a graph, second request")
    assert engine.runner.graph_replays > replays


def test_add_request_refuses_more_than_max_queued_waiting_requests(case):
    from stride_b200 import EngineBusy, SamplingParams
    engine = engine_for(case, "float32", max_queued=2)
    params = SamplingParams(temperature=0.0, max_tokens=3)
    first = [engine.add_request(p, params) for p in case["prompts"][:2]]
    with pytest.raises(EngineBusy, match="max_queued 2"):
        engine.add_request(case["prompts"][2], params)
    engine.step()                                   # both are admitted: nothing waits any more
    third = engine.add_request(case["prompts"][2], params)
    while engine.has_unfinished():
        engine.step()
    for rid, prompt in zip(first + [third], case["prompts"][:3]):
        out = engine.output(rid)
        assert out.finished and out.tokens == plain.greedy_generate(case["cfg"], case["state"]["float32"], prompt, 3, torch.float64)


def test_stop_rules(case):
    from stride_b200 import SamplingParams
    prompt = case["prompts"][-1]
    free_run = plain.greedy_generate(case["cfg"], case["state"]["float32"], prompt, 10, torch.float64)
    engine = engine_for(case, "float32")
    stop_at = free_run[4]
    first = free_run.index(stop_at)
    out = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=10, stop_tokens=[stop_at]))[0]
    assert out.finish_reason == "stop" and out.tokens == free_run[:first], "the stop token itself is not appended"
    # an EOS given to the engine stops too, unless ignored or suppressed by min_tokens
    from stride_b200 import Engine
    e2 = Engine(case["dirs"]["float32"], dtype="float32", block_size=case["page"], num_blocks=64, eos_token_id=free_run[0])
    assert e2.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5))[0].tokens == []
    assert e2.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))[0].tokens == free_run[:5]
    forced = e2.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, min_tokens=2))[0]
    assert len(forced.tokens) >= 2 and forced.tokens[0] != free_run[0]
    with pytest.raises(ValueError):
        engine.add_request([case["cfg"]["vocab_size"]])
    with pytest.raises(ValueError):
        engine.add_request([])
    with pytest.raises(ValueError):
        engine.add_request([1] * case["cfg"]["max_position_embeddings"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_seeded_sampling(case, dtype):
    from stride_b200 import SamplingParams
    # In bfloat16 a repeated prompt must take the same path for the same draws: with the prefix index on, the second
    # run would find the first one's pages and compute only the tail, in a step of another shape, whose rounding
    # differs (float32 is bitwise the same either way, so it keeps the index on).
    engine = engine_for(case, dtype, prefix_caching=dtype == "float32")
    prompt = case["prompts"][1]
    run = lambda **kw: engine.generate([prompt], SamplingParams(max_tokens=16, **kw))[0].tokens
    a, b, c = run(temperature=1.5, seed=1), run(temperature=1.5, seed=1), run(temperature=1.5, seed=2)
    assert a == b and a != c and all(0 <= t < case["cfg"]["vocab_size"] for t in a + c)
    greedy_tokens = run(temperature=0.0)
    assert run(temperature=1.0, top_k=1, seed=3) == greedy_tokens
    assert run(temperature=1e-4, seed=4) == greedy_tokens, "a vanishing temperature must pick the maximum"
    ranked = run(temperature=1.0, top_k=2, top_p=0.9, seed=5)
    assert ranked == run(temperature=1.0, top_k=2, top_p=0.9, seed=5) and len(ranked) == 16
    # the host-ranked path draws from the two most likely tokens only
    logits = plain.forward(case["cfg"], case["state"][dtype], prompt + ranked, torch.float64)
    for i, tok in enumerate(ranked):
        row = logits[len(prompt) - 1 + i]
        third = float(row.topk(3).values[2])
        assert float(row[tok]) >= third - 0.03 * float(row.abs().max())


def test_the_command_line(case, tmp_path):
    prompt = case["prompts"][2]
    want = plain.greedy_generate(case["cfg"], case["state"]["float32"], prompt, 6, torch.float64)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "stride-b200"), "generate", "--model", case["dirs"]["float32"],
                           "--dtype", "float32", "--block-size", str(case["page"]), "--num-blocks", "32", "--temperature", "0",
                           "--max-tokens", "6", "--prompt-tokens", ",".join(map(str, prompt)), "--check-invariants"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert json.loads(proc.stdout.strip().splitlines()[-1])["tokens"] == want


def test_missing_device_or_tensor_on_the_cpu_fails_loudly():
    from stride_b200.csrc import ops
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.add_residual(torch.zeros(2, 2), torch.zeros(2, 2))
