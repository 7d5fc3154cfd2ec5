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


@pytest.fixture(scope="module", params=["A", "B", "D"])
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
    # B and D: prompts that share their first tokens (24 and 40: more than a page, so that later requests find pages
    # of earlier ones in the prefix index); D has the head size and group that the tensor-core kernels take
    lengths = {"A": [1, 7, 16, 33], "B": [3, 25, 41, 57, 72, 90], "D": [3, 41, 57, 72, 90, 150]}[name]
    common = {"A": 0, "B": 24, "D": 40}[name]
    shared = seeded_tokens(common, cfg["vocab_size"], 500)
    out["prompts"] = [(shared[:min(common, n - 1)] + seeded_tokens(n, cfg["vocab_size"], 501 + i))[:n] for i, n in enumerate(lengths)]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_budgets_small_pools_and_resume_give_the_same_tokens(case, dtype):
    """Portions of 5..16 tokens, a pool that cannot hold every request, so that
    requests are preempted and recomputed, with and without the prefix index. In
    bfloat16 (on the configuration whose sizes the tensor-core kernels take: prefill
    attention on tcgen05 reads a prefix that another request wrote, decode attention
    resumes after a preemption) every token is checked against the plain logits of
    the sequence the engine produced."""
    from stride_b200 import SamplingParams
    if dtype == "bfloat16" and case["name"] != "D":
        pytest.skip("bfloat16 runs on the configuration that takes the tensor-core kernels")
    n = case["new_tokens"] + 20
    if dtype == "float32":
        want = [plain.greedy_generate(case["cfg"], case["state"]["float32"], p, n, torch.float64) for p in case["prompts"]]
    longest = max(len(p) for p in case["prompts"]) + n
    pages = -(-longest // case["page"]) + 3
    for prefix_caching in (True, False):
        engine = engine_for(case, dtype, num_blocks=pages, max_batch_tokens=16, max_batch_seqs=4, watermark=0.0,
                            prefix_caching=prefix_caching)
        outs = engine.generate(case["prompts"], SamplingParams(temperature=0.0, max_tokens=n))
        if dtype == "float32":
            assert [o.tokens for o in outs] == want
        else:
            for prompt, out in zip(case["prompts"], outs):
                assert len(out.tokens) == n
                assert_greedy(case, dtype, prompt, out.tokens, f"prompt of {len(prompt)}, prefix index {prefix_caching}")
        m = engine.metrics()
        assert m["preemptions"] > 0, "the pool was meant to be too small"
        assert m["kv_blocks_live"] == 0
        if prefix_caching and case["name"] != "A":
            assert m["prefill_tokens_reused"] > 0, "no request found the shared prefix in the index"


def test_a_poisoned_shared_prefix_shows(case):
    """Negative control of the prefix tests: when the pages that a finished request left in the index are
    overwritten, a later request that adopts them must produce other tokens. If it did not, the tests above could
    not tell whether shared pages are read at all."""
    from stride_b200 import SamplingParams
    if case["name"] == "A":
        pytest.skip("the prompts of this configuration share no prefix")
    dtype = "bfloat16" if case["name"] == "D" else "float32"
    engine = engine_for(case, dtype)
    params = SamplingParams(temperature=0.0, max_tokens=6)
    first, second = case["prompts"][-2], case["prompts"][-1]
    engine.generate([first], params)
    assert engine.cache_stats()["cached"] > 0
    for pages in engine.device_cache.pages:       # every page: the live ones are none, the cached ones hold the prefix
        pages.normal_(0.0, 3.0)
    out = engine.generate([second], params)[0]
    assert out.cached_prompt_tokens >= case["page"], "the second request did not adopt the first one's pages"
    with pytest.raises(AssertionError):
        assert_greedy(case, dtype, second, out.tokens, "poisoned prefix")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_give_the_same_tokens(case, dtype):
    """Decode steps are launched before the tokens of the step before them are read (their token ids travel on the
    device). With that switched off every step waits for its tokens first; both must produce the same tokens and
    events, also for requests that stop on a token in the middle of such a chain, draw with a temperature, or
    reach their limit."""
    from stride_b200 import SamplingParams
    prompts = case["prompts"][-3:]
    free = engine_for(case, dtype, chain_steps=False).generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=24))[0].tokens
    stop_at = free[10]
    params = [SamplingParams(temperature=0.0, max_tokens=24, stop_tokens=[stop_at]), SamplingParams(temperature=0.9, max_tokens=30, seed=11),
              SamplingParams(temperature=0.0, max_tokens=17)]
    runs = {}
    for chain in (False, True):
        engine = engine_for(case, dtype, chain_steps=chain, prefix_caching=False)
        ids = [engine.add_request(p, sp) for p, sp in zip(prompts, params)]
        events = []
        while engine.has_unfinished():
            events += engine.step()
        m = engine.metrics()
        assert (m["chained_steps"] > 5) == chain, m
        assert m["kv_blocks_live"] == 0
        runs[chain] = ([(engine.output(i).tokens, engine.output(i).finish_reason) for i in ids], sorted(events, key=lambda e: e[0]))
    assert runs[True][0][0] == (free[:free.index(stop_at)], "stop")
    assert runs[True] == runs[False]


def test_a_failed_kernel_wait_ends_the_step_with_an_error_and_the_engine_goes_on(case):
    """A wait inside a kernel that cannot be satisfied runs into its limit, records a code in the status word and
    returns (a kernel of this test does exactly that, with a limit of microseconds, on an mbarrier that nothing
    completes). The step whose results come back with that word raises, its requests end with the reason "error",
    the word is cleared, and a request added afterwards runs as if nothing had happened."""
    import ctypes
    from stride_b200 import SamplingParams
    from stride_b200.csrc import build, ops
    lib = build.load_external_library(os.path.join(ROOT, "tests", "kernels", "wait_runs_out.cu"))
    lib.test_wait_runs_out.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    lib.test_wait_runs_out.restype = ctypes.c_int
    engine = engine_for(case, "float32")
    status = ops.status_tensor("cuda")
    returned = torch.full((1,), -1, dtype=torch.int32, device="cuda")

    def run_out(code):
        rc = lib.test_wait_runs_out(status.data_ptr(), code, 100000, returned.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(returned[0]) == 0, "the wait reported success on a barrier that nothing completes"

    # the word by itself: read, reported once, cleared
    run_out(3)
    with pytest.raises(ops.KernelError, match="code 3: matrix product: epilogue"):
        ops.check_kernel_status()
    ops.check_kernel_status()
    # through the engine
    params = SamplingParams(temperature=0.0, max_tokens=4)
    doomed = engine.add_request(case["prompts"][1], params)
    run_out(2)
    with pytest.raises(ops.KernelError, match="code 2"):
        engine.step()
    out = engine.output(doomed)
    assert out.finished and out.finish_reason == "error" and not engine.has_unfinished()
    assert engine.cache_stats()["live"] == 0 and engine.cache_stats()["cached"] == 0, "pages of a failed step must not be shared"
    after = engine.generate([case["prompts"][1]], params)[0]
    assert after.finish_reason == "length"
    assert after.tokens == plain.greedy_generate(case["cfg"], case["state"]["float32"], case["prompts"][1], 4, torch.float64)


def test_a_position_beyond_the_position_tables_is_refused_on_the_host(tmp_models):
    """max_position_embeddings 100 with pages of 16: the block table reaches 112 positions, the rotation tables end
    at 100. The raw step function must refuse position 100 before any kernel reads the tables."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200 import Engine
    cfg = dict(TINY["A"], max_position_embeddings=100)
    folder = write_model_dir(str(tmp_models / "short_tables"), cfg, seeded_state(cfg, 3), torch.float32)
    engine = Engine(folder, dtype="float32", block_size=16, num_blocks=16, max_model_len=4096)
    assert engine.max_model_len == 100
    engine.cache.open(7, "t")
    assert engine.cache.ensure(7, 112, 0)
    tokens = seeded_tokens(100, cfg["vocab_size"], 1)
    assert engine.forward([(7, tokens, 0, [99])]).shape == (1, cfg["vocab_size"])
    with pytest.raises(ValueError, match="position 100"):
        engine.forward([(7, [5], 100, [0])])
    with pytest.raises(ValueError, match="max_model_len is 100"):
        engine.forward([(7, tokens[:12], 95, [0])])
    engine.cache.close(7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_alone_is_prefilled_in_full_portions_from_a_graph(case, dtype):
    """One request whose prompt is several token budgets long: every portion but the last fills the budget and is
    replayed from the graph captured for such portions; the tokens are the plain ones."""
    from stride_b200 import SamplingParams
    prompt = seeded_tokens(3 * 16 + 5, case["cfg"]["vocab_size"], 777)
    engine = engine_for(case, dtype, max_batch_tokens=16, max_batch_seqs=4)
    out = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6))[0]
    assert_greedy(case, dtype, prompt, out.tokens, "full portions from a graph")
    if case["name"] == "D":
        # portions of 48 tokens: above 16 rows the bfloat16 products are the library's and the prefill attention on
        # tcgen05 runs, from the captured graph, at positions 48 and 96
        wide = engine_for(case, dtype, max_batch_tokens=48, max_batch_seqs=4)
        long_prompt = seeded_tokens(3 * 48 + 7, case["cfg"]["vocab_size"], 778)
        more = wide.generate([long_prompt], SamplingParams(temperature=0.0, max_tokens=6))[0]
        assert_greedy(case, dtype, long_prompt, more.tokens, "portions of 48 from a graph")
        assert ("portion", 0) in wide.runner._graphs and wide.runner.graph_replays >= 3
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
    cold = run(temperature=1e-4, seed=4)
    if dtype == "float32":
        assert cold == greedy_tokens, "a vanishing temperature must pick the maximum"
    else:
        # two logits that bfloat16 cannot tell apart may fall either way: every token must be a maximum of the plain
        # logits within rounding, and the run may part from the greedy one only at such a near-tie
        assert_greedy(case, dtype, prompt, cold, "a vanishing temperature must pick the maximum")
    ranked = run(temperature=1.0, top_k=2, top_p=0.9, seed=5)
    assert ranked == run(temperature=1.0, top_k=2, top_p=0.9, seed=5) and len(ranked) == 16
    # a draw with top_k 2 (on the device by default) comes from the two most likely tokens only
    logits = plain.forward(case["cfg"], case["state"][dtype], prompt + ranked, torch.float64)
    for i, tok in enumerate(ranked):
        row = logits[len(prompt) - 1 + i]
        third = float(row.topk(3).values[2])
        assert float(row[tok]) >= third - 0.03 * float(row.abs().max())


def test_top_k_and_nucleus_rows_are_drawn_on_the_device_as_on_the_host(case):
    """The same seeded requests with the cuts applied by the device kernel and by the host sampler (from logits brought
    back): the same tokens (float32: both see bitwise the same logits, and one uniform number is drawn per token either
    way), and on the device such rows no longer keep decode steps from being launched ahead."""
    from stride_b200 import SamplingParams
    prompts = [case["prompts"][1], case["prompts"][2], case["prompts"][0]]
    params = [SamplingParams(max_tokens=24, temperature=0.9, top_k=7, seed=21), SamplingParams(max_tokens=24, temperature=1.3, top_p=0.8, seed=22),
              SamplingParams(max_tokens=24, temperature=1.0, top_k=40, top_p=0.95, seed=23, min_tokens=3)]
    on_device = engine_for(case, "float32", device_ranking=True)
    on_host = engine_for(case, "float32", device_ranking=False)
    a = [o.tokens for o in on_device.generate(prompts, params)]
    b = [o.tokens for o in on_host.generate(prompts, params)]
    assert a == b
    assert all(len(t) == 24 for t in a) and len({tuple(t) for t in a}) == 3
    assert on_device.metrics()["chained_steps"] > 0 and on_host.metrics()["chained_steps"] == 0
    assert on_device.d2h_bytes < on_host.d2h_bytes, "the host path brings the logits of ranked rows back"


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
