"""The scheduler's decisions with a fake model (no GPU): every decode slot is
answered with token 7, as the reference's scheduling tests do
(crates/stride-sched/tests/scheduling.rs:25-35)."""

import random

import pytest

from stride_b200.cache import CacheManager, runtime

rt = runtime()
Interactive, Batch, Background = rt.ServiceClass.Interactive, rt.ServiceClass.Batch, rt.ServiceClass.Background


def make(pages=64, page=16, slots=32, prefix=True, **cfg):
    cache = CacheManager(page, [(pages, 0)], slots, prefix)
    sched = rt.Scheduler(rt.SchedulerConfig(**cfg), cache)
    return sched, cache


def greedy(n):
    return rt.SamplingParams.greedy(n)


def run_step(sched, cache, now, token=7):
    """One engine iteration with the fake model. Returns (batch, finished)."""
    batch = sched.step(now)
    cache.check_invariants()
    step_batch = sched.build_batch(batch)          # also checks that every table covers its tokens
    assert step_batch.num_tokens == batch.num_tokens
    sched.after_step(batch)
    outputs = [(seq, token) for seq in step_batch.row_requests()]
    finished = sched.on_tokens(outputs, now + 10)
    cache.check_invariants()
    return batch, finished


def drain(sched, cache, now=0, limit=10000):
    done = []
    for _ in range(limit):
        if sched.idle:
            return done, now
        _, fin = run_step(sched, cache, now)
        done += fin
        now += 1000
    raise AssertionError("the scheduler did not drain")


def test_admission_refusals():
    sched, _ = make(max_model_len=64)
    with pytest.raises(ValueError, match="empty"):
        sched.admit(1, "t", [], greedy(4))
    with pytest.raises(ValueError, match="max_model_len"):
        sched.admit(2, "t", [1] * 64, greedy(4))
    bad = rt.SamplingParams(temperature=3.0)
    with pytest.raises(ValueError, match="temperature"):
        sched.admit(3, "t", [1, 2], bad)
    small, _ = make(pages=4, max_model_len=4096)
    with pytest.raises(ValueError, match="pages"):
        small.admit(4, "t", [1] * 100, greedy(4))
    assert sched.num_waiting == 0 and small.num_waiting == 0


def test_one_request_prefill_then_decodes_then_length():
    sched, cache = make()
    seq = sched.admit(1, "t", list(range(20)), greedy(3))
    b, fin = run_step(sched, cache, 0)
    assert [(c.seq, c.start, c.len) for c in b.prefill] == [(seq, 0, 20)] and b.decode == [] and not fin
    s = sched.sequence(seq)
    assert s.state == rt.SeqState.Decoding and s.output == [7] and s.kv_len == 20 and s.total_len == 21
    b, fin = run_step(sched, cache, 1000)
    assert b.decode == [seq] and b.prefill == [] and not fin
    b, fin = run_step(sched, cache, 2000)
    assert len(fin) == 1 and fin[0].reason == rt.FinishReason.Length and fin[0].output == [7, 7, 7]
    assert sched.idle and cache.stats()["live"] == 0
    # 22 tokens had keys written (the last sampled token never ran): one full page is reusable
    assert cache.stats()["cached"] == 1


def test_the_token_budget_holds_and_long_prompts_are_cut():
    sched, cache = make(pages=256, max_batch_tokens=128, max_model_len=4096)
    seq = sched.admit(1, "t", [3] * 1024, greedy(2))
    chunks = []
    for step in range(20):
        b, _ = run_step(sched, cache, step * 1000)
        assert b.num_tokens <= 128
        chunks += [(c.start, c.len) for c in b.prefill]
        if sched.idle:
            break
    assert len(chunks) == 8 and chunks[0] == (0, 128) and chunks[-1] == (896, 128)
    assert sched.idle


def test_no_chunking_waits_for_room():
    sched, cache = make(pages=256, max_batch_tokens=64, chunked_prefill=False, max_model_len=4096)
    with pytest.raises(ValueError, match="chunked prefill is off"):
        sched.admit(1, "t", [1] * 100, greedy(2))
    a = sched.admit(2, "t", [1] * 40, greedy(2))
    b_ = sched.admit(3, "t", [2] * 40, greedy(2))
    b, _ = run_step(sched, cache, 0)
    assert [c.seq for c in b.prefill] == [a], "the second prompt does not fit the budget whole and must wait"
    b, _ = run_step(sched, cache, 1000)
    assert b.decode == [a] and [c.seq for c in b.prefill] == [b_]


def test_decodes_continue_while_a_long_prompt_is_prefilled():
    sched, cache = make(pages=256, max_batch_tokens=64, max_model_len=4096)
    short = sched.admit(1, "t", [1] * 8, greedy(50))
    run_step(sched, cache, 0)
    long = sched.admit(2, "t", [2] * 300, greedy(2))
    for step in range(1, 5):
        b, _ = run_step(sched, cache, step * 1000)
        assert b.decode == [short], "the running decode was displaced"
        assert [c.seq for c in b.prefill] == [long] and b.prefill[0].len == 63
        assert b.num_tokens == 64


def test_admission_is_ranked_by_slack_not_by_class():
    sched, cache = make(max_batch_seqs=1)
    old_background = sched.admit(1, "t", [1] * 4, greedy(1), Background, 0)
    fresh_interactive = sched.admit(2, "t", [2] * 4, greedy(1), Interactive, 119_900_000)
    assert sched.slack_us(old_background, 119_900_000) < sched.slack_us(fresh_interactive, 119_900_000)
    b, _ = run_step(sched, cache, 119_900_000)
    assert [c.seq for c in b.prefill] == [old_background]
    # and the other way round when both are fresh
    sched, cache = make(max_batch_seqs=1)
    bg = sched.admit(1, "t", [1] * 4, greedy(1), Background, 0)
    ia = sched.admit(2, "t", [2] * 4, greedy(1), Interactive, 0)
    b, _ = run_step(sched, cache, 10)
    assert [c.seq for c in b.prefill] == [ia]
    assert rt.ttft_budget_us(Interactive) == 500_000 and rt.itl_budget_us(Batch) == 200_000


def test_preemption_takes_the_most_slack_and_resume_recomputes():
    # 8 pages of 4 tokens; two requests that both grow until the pool is full
    sched, cache = make(pages=8, page=4, prefix=False, watermark=0.0, max_model_len=64)
    a = sched.admit(1, "t", [1] * 10, greedy(12), Interactive, 0)
    b_ = sched.admit(2, "t", [2] * 10, greedy(12), Background, 0)
    preempted_at = None
    for step in range(40):
        batch, _ = run_step(sched, cache, step * 1000)
        if batch.preempted:
            preempted_at = step
            assert batch.preempted == [b_], "the background request has the most slack and must yield"
            assert b_ not in batch.decode, "a preempted request must leave the batch being built"
            s = sched.sequence(b_)
            assert s.state == rt.SeqState.Swapped and s.kv_len == 0 and s.preemptions == 1
            assert not cache.has(b_)
            break
    assert preempted_at is not None
    done, _ = drain(sched, cache, 100_000)
    outs = {f.seq: f.output for f in done}
    assert outs[a] == [7] * 12 and outs[b_] == [7] * 12
    assert sched.metrics()["preemptions"] >= 1 and cache.stats()["live"] == 0


def test_a_prefill_waits_when_pages_run_out_and_goes_on_when_they_return():
    sched, cache = make(pages=8, page=4, prefix=False, watermark=0.0, max_batch_tokens=8, max_model_len=64)
    a = sched.admit(1, "t", [1] * 26, greedy(2))
    b, _ = run_step(sched, cache, 0)
    assert [(c.start, c.len) for c in b.prefill] == [(0, 8)]
    cache.open(999, "someone else")          # pages taken behind the scheduler's back
    assert cache.ensure(999, 20)
    for step in range(1, 4):
        b, _ = run_step(sched, cache, step * 1000)
        assert b.is_empty() and not b.preempted, "nothing fits and nobody can be preempted: the step is empty"
        assert sched.sequence(a).state == rt.SeqState.Prefilling and sched.sequence(a).kv_len == 8
    cache.close(999)
    done, _ = drain(sched, cache, 10_000)
    assert [f.seq for f in done] == [a] and done[0].output == [7, 7]


def test_a_short_request_may_start_while_a_longer_one_waits_for_pages():
    # Request a is in the middle of its prompt when the pool fills up; a later, shorter
    # request b still fits, starts and decodes; a goes on once pages return.
    sched, cache = make(pages=8, page=4, prefix=False, watermark=0.0, max_batch_tokens=12, max_model_len=64)
    a = sched.admit(1, "t", [1] * 24, greedy(2))
    b, _ = run_step(sched, cache, 0)
    assert [(c.seq, c.len) for c in b.prefill] == [(a, 12)]
    cache.open(999, "someone else")
    assert cache.ensure(999, 12)             # 3 + 3 pages held, 2 left: a needs 3 more and must wait
    b_ = sched.admit(2, "t", [2] * 4, greedy(20))
    b, _ = run_step(sched, cache, 1000)
    assert [(c.seq, c.len) for c in b.prefill] == [(b_, 4)], "the short request fits (1 page + 1 reserve) and starts"
    cache.close(999)
    cache.open(998, "someone else")
    assert cache.ensure(998, 8)              # a: 3, b: 1, foreign: 2 -> 2 left
    b, _ = run_step(sched, cache, 2000)      # b decodes; a still cannot get 3 pages (+1 reserve)
    assert b.decode == [b_] and not b.prefill
    cache.close(998)
    done, _ = drain(sched, cache, 3000)
    assert sorted(f.seq for f in done) == [a, b_]


def test_stop_and_cancel_release_everything():
    sched, cache = make()
    a = sched.admit(1, "t", list(range(40)), greedy(8))
    b_ = sched.admit(2, "t", list(range(100, 130)), greedy(8))
    run_step(sched, cache, 0)
    f = sched.stop(a)
    assert f.reason == rt.FinishReason.Stop and f.output == [7], "a stop does not append another token"
    assert sched.stop(a) is None
    fin = sched.cancel(2)
    assert [x.seq for x in fin] == [b_] and fin[0].reason == rt.FinishReason.Cancelled
    assert sched.idle and cache.stats()["live"] == 0 and cache.free_slots == cache.slot_capacity
    cache.check_invariants()


def test_prefix_reuse_through_the_scheduler():
    sched, cache = make(pages=64, page=16)
    prompt = list(range(64))
    sched.admit(1, "acme", prompt, greedy(1))
    drain(sched, cache)
    assert sched.metrics()["prefill_tokens_reused"] == 0
    second = sched.admit(2, "acme", prompt, greedy(1))
    b, _ = run_step(sched, cache, 0)
    assert [(c.start, c.len, c.cached) for c in b.prefill] == [(48, 16, 48)]
    third = sched.admit(3, "other", prompt, greedy(1))
    b, _ = run_step(sched, cache, 1000)
    assert [(c.seq, c.start) for c in b.prefill] == [(third, 0)], "another tenant must not share pages"
    m = sched.metrics()
    assert m["prefill_tokens_reused"] == 48 and 0 < m["prefill_reuse_rate"] < 1


def test_a_finished_request_does_not_publish_a_page_with_an_unwritten_slot():
    # 15-token prompt + 1 generated token = 16 tokens = one page, but the last token never ran
    sched, cache = make(pages=8, page=16)
    sched.admit(1, "t", list(range(15)), greedy(1))
    drain(sched, cache)
    assert cache.stats()["cached"] == 0
    seq = sched.admit(2, "t", list(range(15)) + [7, 1, 2], greedy(1))
    b, _ = run_step(sched, cache, 0)
    assert b.prefill[0].start == 0 and b.prefill[0].cached == 0


def test_generation_stops_at_max_model_len():
    sched, cache = make(max_model_len=12)
    seq = sched.admit(1, "t", [1] * 10, greedy(50))
    done, _ = drain(sched, cache)
    assert len(done) == 1 and done[0].reason == rt.FinishReason.Length and len(done[0].output) == 2


def test_invariants_hold_through_many_rounds_of_pressure_and_the_pool_drains():
    rng = random.Random(7)
    sched, cache = make(pages=24, page=8, slots=6, max_batch_tokens=48, max_batch_seqs=4, max_model_len=160)
    now, request, finished = 0, 0, 0
    shared = [rng.randrange(50) for _ in range(24)]
    for round_ in range(60):
        for _ in range(rng.randint(0, 2)):
            request += 1
            prompt = shared[:rng.choice([0, 8, 16, 24])] + [rng.randrange(50) for _ in range(rng.randint(1, 40))]
            klass = rng.choice([Interactive, Batch, Background])
            sched.admit(request, rng.choice(["a", "b"]), prompt, greedy(rng.randint(1, 20)), klass, now)
        batch, fin = run_step(sched, cache, now)
        assert batch.num_tokens <= 48 and batch.num_seqs <= 4
        assert len(set(batch.decode) | {c.seq for c in batch.prefill}) == batch.num_seqs, "a request was placed twice"
        assert not (set(batch.preempted) & (set(batch.decode) | {c.seq for c in batch.prefill}))
        finished += len(fin)
        if round_ % 9 == 4 and sched.running_ids:
            finished += len(sched.cancel(sched.sequence(sched.running_ids[0]).request))
        now += 7000
    done, _ = drain(sched, cache, now)
    finished += len(done)
    assert finished == request
    m = sched.metrics()
    assert m["admitted"] == request and m["finished"] == request
    assert m["preemptions"] > 0, "the scenario was meant to run out of pages"
    assert m["prefill_tokens_reused"] > 0, "the scenario was meant to hit the prefix index"
    s = cache.stats()
    assert s["live"] == 0 and s["free"] + s["cached"] == s["capacity"] and cache.free_slots == cache.slot_capacity


def test_the_step_invariant_can_fail():
    sched, cache = make()
    sched.admit(1, "t", [1] * 20, greedy(2))
    run_step(sched, cache, 0)
    cache.corrupt_for_test(0, 2)
    with pytest.raises(rt.InvariantError):
        run_step(sched, cache, 1000)
