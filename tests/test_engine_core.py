"""The host side of the engine's step in C++ (``EngineCore``) against a plain Python loop over the same scheduler,
samplers and cache manager, with a stand-in for the device (pseudo-logits that depend on the whole context, and an
emulation of the device sampler): same events in the same order, same outputs, same counters, under small pools
(preemption and resume), stop rules, suppression of the end token, ranking on the host, cancellation. No GPU."""

import hashlib
import random

import numpy as np
import pytest

from stride_b200.csrc.build import load_runtime

rt = load_runtime()
VOCAB, EOS, PAGE = 48, 3, 4
BASE_SEED = 0x57219A3C11FF0042


def pseudo_logits(context) -> np.ndarray:
    """float32 [VOCAB] that depends on every token of the context (so a wrong position or a lost token shows)."""
    digest = hashlib.sha256(np.asarray(context, dtype=np.int32).tobytes()).digest()
    rng = np.random.default_rng(int.from_bytes(digest[:8], "little"))
    return (rng.standard_normal(VOCAB) * 2.0).astype(np.float32)


def device_sampler(logits, temperature, uniform, suppress) -> int:
    """What the sampling kernel does with one row: suppression, first maximum at temperature 0, else the softmax of
    logits / temperature walked in vocabulary order up to uniform * total."""
    row = logits.astype(np.float64).copy()
    if suppress >= 0:
        row[suppress] = -np.inf
    if temperature == 0.0:
        return int(np.argmax(row))
    p = np.exp((row - row.max()) / temperature)
    target = uniform * p.sum()
    return int(min(np.searchsorted(np.cumsum(p), target, side="left"), VOCAB - 1))


def make_scheduler(pages, max_batch_tokens=16, max_batch_seqs=4, max_model_len=96):
    cache = rt.CacheManager(PAGE, [(pages, 0)], max_batch_seqs, True)
    sched = rt.Scheduler(rt.SchedulerConfig(max_batch_seqs, max_batch_tokens, max_model_len, 0.0, True), cache)
    return cache, sched


def row_logits(sched, batch):
    """Logits of every wanted row of a step batch, in row order, from the sequences' own tokens."""
    rows = []
    for seq, tokens, position, want in batch.items():
        history = list(sched.sequence(seq).tokens)
        assert history[position:position + len(tokens)] == list(tokens)
        rows += [pseudo_logits(history[:position + w + 1]) for w in want]
    return rows


class PythonLoop:
    """The engine's step as the Python entry point runs it, with the stand-in device."""

    def __init__(self, sched, cache, extra_stops=(), max_queued=1024):
        self.sched, self.cache, self.extra, self.max_queued = sched, cache, tuple(extra_stops), max_queued
        self.active, self.outputs, self.next_request = {}, {}, 1

    def add_request(self, prompt, params, now):
        if self.sched.num_waiting >= self.max_queued:
            raise rt.EngineBusy("busy")
        for t in prompt:
            if not 0 <= t < VOCAB:
                raise ValueError("vocabulary")
        if self.extra:
            params = rt.SamplingParams(params.temperature, params.top_p, params.top_k, params.max_tokens, params.min_tokens,
                                       list(params.stop_tokens) + [e for e in self.extra if e not in params.stop_tokens],
                                       params.seed, params.ignore_eos)
        rid = self.next_request
        seq = self.sched.admit(rid, "default", list(prompt), params, rt.ServiceClass.Interactive, now)
        self.next_request += 1
        sampler = rt.Sampler(params, EOS, (BASE_SEED + rid) & 0xFFFFFFFFFFFFFFFF)
        self.active[seq] = (rid, sampler)
        self.outputs[rid] = {"tokens": [], "finished": False, "reason": None, "seed": sampler.effective_seed}
        return rid

    def cancel(self, rid):
        events = []
        for f in self.sched.cancel(rid):
            events.append((f.request, None, "Cancelled"))
            self._retire(f.seq, "Cancelled")
        return events

    def _retire(self, seq, reason):
        rid, _ = self.active.pop(seq)
        self.outputs[rid].update(finished=True, reason=reason)
        self.sched.forget(seq)

    def step(self, now):
        scheduled = self.sched.step(now)
        if scheduled.is_empty():
            return None
        batch = self.sched.build_batch(scheduled)
        logits = row_logits(self.sched, batch)
        seqs = batch.row_requests()
        tokens = []
        for r, seq in enumerate(seqs):
            rid, sampler = self.active[seq]
            p = sampler.params
            generated = len(self.outputs[rid]["tokens"])
            suppress = sampler.suppressed_token(generated)
            if p.needs_ranking():
                tokens.append(None)
            elif p.is_greedy():
                tokens.append(device_sampler(logits[r], 0.0, 0.0, suppress))
            else:
                tokens.append(device_sampler(logits[r], float(np.float32(p.temperature)), sampler.next_uniform(), suppress))
        for r, seq in enumerate(seqs):
            if tokens[r] is None:
                rid, sampler = self.active[seq]
                tokens[r] = sampler.sample(logits[r], len(self.outputs[rid]["tokens"]))
        self.sched.after_step(scheduled)
        events, sampled, stopped = [], [], []
        for seq, token in zip(seqs, tokens):
            rid, sampler = self.active[seq]
            if sampler.is_stop(token):
                stopped.append(seq)
            else:
                sampled.append((seq, token))
                self.outputs[rid]["tokens"].append(token)
                events.append((rid, token, None))
        finished = self.sched.on_tokens(sampled, now)
        for seq in stopped:
            self.sched.stop(seq)
            events.append((self.active[seq][0], None, "Stop"))
            self._retire(seq, "Stop")
        for f in finished:
            events.append((f.request, None, "Length"))
            self._retire(f.seq, "Length")
        return events


class CoreLoop:
    """The same step through ``EngineCore``: begin_step, the stand-in device, finish_step."""

    def __init__(self, sched, cache, extra_stops=(), max_queued=1024, rows=8):
        self.sched, self.cache = sched, cache
        self.core = rt.EngineCore(sched, EOS, list(extra_stops), BASE_SEED, max_queued, VOCAB)
        self.temperature = np.zeros(rows, dtype=np.float32)
        self.uniform = np.zeros(rows, dtype=np.float32)
        self.suppress = np.zeros(rows, dtype=np.int32)

    def add_request(self, prompt, params, now):
        return self.core.add_request(list(prompt), params, "default", rt.ServiceClass.Interactive, now)

    def cancel(self, rid):
        return [(e.request, e.token, e.reason.name) for e in self.core.cancel(rid)]

    def step(self, now):
        if not self.core.begin_step(now):
            return None
        batch = self.core.batch()
        logits = row_logits(self.sched, batch)
        assert list(self.core.rows()) == list(batch.row_requests())
        ranked = self.core.prepare_sampling(self.temperature, self.uniform, self.suppress)
        n = len(logits)
        tokens = np.array([device_sampler(logits[r], float(self.temperature[r]), float(self.uniform[r]), int(self.suppress[r]))
                           for r in range(n)], dtype=np.int32)
        ranked_logits = np.stack([logits[r] for r in ranked]) if ranked else None
        events = self.core.finish_step(tokens, ranked, ranked_logits, now)
        return [(e.request, e.token, None if e.reason == rt.FinishReason.NotFinished else e.reason.name) for e in events]


def ranked_draw(logits, temperature, uniform, suppress, top_k, top_p) -> int:
    """What a device that ranks does with a row that has cuts: the host sampler's rule with float32 sums in its order
    (crates/stride-backend/src/sampler.rs:88-146), the uniform number given instead of drawn."""
    work = logits.astype(np.float32).copy()
    if suppress >= 0:
        work[suppress] = -np.inf
    if abs(temperature - 1.0) > 1.1920929e-07:
        work = work / np.float32(temperature)
    e = np.exp(work - work.max()).astype(np.float32)
    total = np.float32(0)
    for v in e:
        total = np.float32(total + v)
    probs = (e / total).astype(np.float32)
    kept = rt.rank_head(probs, top_k if top_k > 0 else None, float(top_p))
    mass = np.float32(0)
    for i in kept:
        mass = np.float32(mass + probs[i])
    target = np.float32(np.float32(uniform) * mass)
    for i in kept:
        target = np.float32(target - probs[i])
        if target <= 0:
            return int(i)
    return int(kept[-1])


class DeviceRankLoop(CoreLoop):
    """``EngineCore`` with a device that draws the ranked rows too: the core hands out their cuts and a uniform number
    and gets every token back; nothing is ranked in finish_step."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.core.set_device_ranks(True)
        self.top_k = np.zeros(len(self.temperature), dtype=np.int32)
        self.top_p = np.ones(len(self.temperature), dtype=np.float32)
        self.drawn_with_cuts = 0

    def step(self, now):
        if not self.core.begin_step(now):
            return None
        logits = row_logits(self.sched, self.core.batch())
        ranked = self.core.prepare_sampling(self.temperature, self.uniform, self.suppress, self.top_k, self.top_p)
        assert list(ranked) == []
        tokens = []
        for r in range(len(logits)):
            t, u, ban, k, p = float(self.temperature[r]), float(self.uniform[r]), int(self.suppress[r]), int(self.top_k[r]), float(self.top_p[r])
            if t > 0 and (k > 0 or p < 1.0):
                tokens.append(ranked_draw(logits[r], t, u, ban, k, p))
                self.drawn_with_cuts += 1
            else:
                tokens.append(device_sampler(logits[r], t, u, ban))
        events = self.core.finish_step(np.array(tokens, dtype=np.int32), [], None, now)
        return [(e.request, e.token, None if e.reason == rt.FinishReason.NotFinished else e.reason.name) for e in events]


def random_params(rng):
    kind = rng.choice(["greedy", "greedy", "temperature", "seeded", "top_k", "top_p", "min_tokens", "stops", "ignore_eos"])
    max_tokens = rng.randint(1, 12)
    if kind == "greedy":
        return rt.SamplingParams(0.0, 1.0, None, max_tokens, 0, [], None, False)
    if kind == "temperature":
        return rt.SamplingParams(rng.choice([0.7, 1.0, 1.5]), 1.0, None, max_tokens, 0, [], None, False)
    if kind == "seeded":
        return rt.SamplingParams(0.9, 1.0, None, max_tokens, 0, [], rng.randrange(1 << 40), False)
    if kind == "top_k":
        return rt.SamplingParams(1.0, 1.0, rng.choice([1, 3, 8]), max_tokens, 0, [], None, False)
    if kind == "top_p":
        return rt.SamplingParams(1.2, rng.choice([0.5, 0.9]), rng.choice([None, 6]), max_tokens, 0, [], None, False)
    if kind == "min_tokens":
        return rt.SamplingParams(0.0, 1.0, None, max_tokens, rng.randint(0, max_tokens), [], None, False)
    if kind == "stops":
        return rt.SamplingParams(1.0, 1.0, None, max_tokens, 0, [rng.randrange(VOCAB) for _ in range(6)], None, False)
    return rt.SamplingParams(1.0, 1.0, None, max_tokens, 0, [], None, True)


@pytest.mark.parametrize("seed", range(8))
def test_core_and_python_loop_agree_event_by_event(seed):
    rng = random.Random(seed)
    pages = rng.choice([14, 18, 40])                   # small pools: requests are preempted and recomputed
    extra = rng.choice([(), (5, 9)])
    loops = []
    for cls in (PythonLoop, CoreLoop):
        cache, sched = make_scheduler(pages)
        loops.append(cls(sched, cache, extra_stops=extra))
    arrivals = sorted((rng.randint(0, 40), [rng.randrange(VOCAB) for _ in range(rng.randint(1, 30))], random_params(random.Random(seed * 100 + i)))
                      for i in range(14))
    cancel_at = {rng.randint(5, 45): rng.randint(1, 14) for _ in range(3)}
    now, step, idle, preempted = 0, 0, 0, 0
    while step < 400:
        for at, prompt, params in arrivals:
            if at == step:
                ids = []
                for loop in loops:
                    try:
                        ids.append(loop.add_request(prompt, params, now))
                    except ValueError as e:        # a request that can never fit is refused by both
                        ids.append(type(e).__name__)
                assert ids[0] == ids[1]
        if step in cancel_at:
            a, b = (loop.cancel(cancel_at[step]) for loop in loops)
            assert a == b
        a, b = (loop.step(now) for loop in loops)
        assert a == b, f"step {step}: events differ"
        for loop in loops:
            loop.cache.check_invariants()
        idle = idle + 1 if a is None else 0
        now += 1000
        step += 1
        if idle > 3 and step > 45:
            break
    py, core = loops
    assert not py.active and not core.core.has_unfinished(), "requests were left unfinished"
    for rid, out in py.outputs.items():
        rec = core.core.record(rid)
        assert rec.tokens == out["tokens"] and rec.finished == out["finished"] and rec.seed == out["seed"]
        assert (rec.reason.name if rec.finished else None) == out["reason"]
    assert dict(py.sched.metrics()) == dict(core.sched.metrics())
    assert py.cache.stats(0) == core.cache.stats(0)
    assert core.cache.stats(0)["live"] == 0


@pytest.mark.parametrize("seed", range(6))
def test_a_device_that_ranks_gets_cuts_and_uniforms_and_changes_no_event(seed):
    rng = random.Random(100 + seed)
    pages = rng.choice([14, 18, 40])
    loops = []
    for cls in (CoreLoop, DeviceRankLoop):
        cache, sched = make_scheduler(pages)
        loops.append(cls(sched, cache))
    arrivals = sorted((rng.randint(0, 30), [rng.randrange(VOCAB) for _ in range(rng.randint(1, 30))], random_params(random.Random(seed * 77 + i)))
                      for i in range(14))
    now, step, idle = 0, 0, 0
    while step < 400:
        for at, prompt, params in arrivals:
            if at == step:
                ids = []
                for loop in loops:
                    try:
                        ids.append(loop.add_request(prompt, params, now))
                    except ValueError as e:
                        ids.append(type(e).__name__)
                assert ids[0] == ids[1]
        a, b = (loop.step(now) for loop in loops)
        assert a == b, f"step {step}: events differ"
        idle = idle + 1 if a is None else 0
        now += 1000
        step += 1
        if idle > 3 and step > 35:
            break
    host, device = loops
    assert not host.core.has_unfinished() and not device.core.has_unfinished()
    assert device.core.device_ranks and not host.core.device_ranks
    if seed == 0:
        assert sum(l.drawn_with_cuts for l in [device]) > 0, "no row had a cut: the test says nothing"


def test_preemption_happens_in_the_small_pools_and_outputs_survive_it():
    cache, sched = make_scheduler(pages=12, max_batch_tokens=8)
    loop = CoreLoop(sched, cache)
    params = rt.SamplingParams(0.0, 1.0, None, 10, 0, [], None, True)
    prompts = [[(7 * i + j) % VOCAB for j in range(14)] for i in range(3)]
    ids = [loop.add_request(p, params, 0) for p in prompts]
    now = 0
    while loop.core.has_unfinished():
        loop.step(now)
        cache.check_invariants()
        now += 1000
        assert now < 10_000_000
    assert sched.metrics()["preemptions"] > 0, "the pool was meant to be too small"
    for rid, prompt in zip(ids, prompts):             # greedy on context-determined logits: the plain continuation
        want, ctx = [], list(prompt)
        for _ in range(10):
            want.append(int(np.argmax(pseudo_logits(ctx))))
            ctx.append(want[-1])
        assert loop.core.record(rid).tokens == want


def test_refusals_and_misuse_are_errors():
    cache, sched = make_scheduler(pages=40)
    core = rt.EngineCore(sched, EOS, [], BASE_SEED, 2, VOCAB)
    params = rt.SamplingParams(0.0, 1.0, None, 4, 0, [], None, False)
    with pytest.raises(ValueError, match="vocabulary"):
        core.add_request([1, VOCAB], params)
    with pytest.raises(ValueError):
        core.add_request([], params)
    a, b = core.add_request([1, 2], params), core.add_request([3], params)
    assert (a, b) == (1, 2) and core.record(a).seed == (BASE_SEED + 1) & 0xFFFFFFFFFFFFFFFF
    with pytest.raises(rt.EngineBusy, match="max_queued 2"):
        core.add_request([4], params)
    with pytest.raises(RuntimeError):
        core.batch()
    assert core.begin_step(0)
    with pytest.raises(RuntimeError):
        core.begin_step(0)
    with pytest.raises(ValueError, match="one token per wanted row"):
        core.finish_step(np.zeros(5, dtype=np.int32))
    with pytest.raises(IndexError):
        core.record(99)
    with pytest.raises(ValueError):
        rt.EngineCore(sched, EOS, [], BASE_SEED, 0, VOCAB)
    core.abandon_step()
    assert core.num_live == 2
    events = core.cancel(a)
    assert [(e.request, e.token, e.reason.name) for e in events] == [(a, None, "Cancelled")] and core.record(a).finished
    core.forget(a)
    with pytest.raises(IndexError):
        core.record(a)


# --------------------------------------------------------------------------------------- steps launched ahead
class ChainLoop(CoreLoop):
    """The loop with the next step launched before the tokens of the open one are read. The stand-in device keeps
    the tokens it has drawn (as the device does) and feeds them to the chained step's rows; the host reads them
    afterwards. `launches` records, per device step, whether it was launched ahead."""

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.pending = None            # (tokens drawn by the step launched ahead, in row order)
        self.launches = []

    def _run_on_device(self, batch, feed):
        """Logits and device-drawn tokens of a batch; `feed[r]`, when given, replaces the single token of item r."""
        rows = []
        for r, (seq, tokens, position, want) in enumerate(batch.items()):
            history = list(self.sched.sequence(seq).tokens) if self.sched.sequence(seq) is not None else None
            if feed is not None:
                # the chained step: its context is what the host knew at launch time plus the token fed on the device
                history = self._history_at_launch[seq] + [int(feed[r])]
                assert position == len(history) - 1
            rows += [pseudo_logits(history[:position + w + 1]) for w in want]
        return rows

    def step(self, now):
        core = self.core
        if not core.begin_step(now):
            return None
        if core.launched_ahead():
            tokens = self.pending                       # launched and drawn already
            self.pending = None
            self.launches.append("ahead")
        else:
            batch = core.batch()
            logits = row_logits(self.sched, batch)
            ranked = core.prepare_sampling(self.temperature, self.uniform, self.suppress)
            tokens = np.array([device_sampler(logits[r], float(self.temperature[r]), float(self.uniform[r]), int(self.suppress[r]))
                               for r in range(len(logits))], dtype=np.int32)
            self.launches.append("now")
            if ranked:
                ranked_logits = np.stack([logits[r] for r in ranked])
                events = core.finish_step(tokens, ranked, ranked_logits, now)
                return [(e.request, e.token, None if e.reason == rt.FinishReason.NotFinished else e.reason.name) for e in events]
        # the tokens of the open step are on the device now, not yet on the host: launch the step after it
        if core.chain_step():
            nxt = core.next_batch()
            self._history_at_launch = {seq: list(self.sched.sequence(seq).tokens) for seq, _t, _p, _w in nxt.items()}
            core.prepare_next_sampling(self.temperature, self.uniform, self.suppress)
            logits = self._run_on_device(nxt, feed=tokens)
            self.pending = np.array([device_sampler(logits[r], float(self.temperature[r]), float(self.uniform[r]), int(self.suppress[r]))
                                     for r in range(len(logits))], dtype=np.int32)
        events = core.finish_step(tokens, [], None, now)
        return [(e.request, e.token, None if e.reason == rt.FinishReason.NotFinished else e.reason.name) for e in events]


@pytest.mark.parametrize("seed", range(10))
def test_steps_launched_ahead_change_no_token(seed):
    """Every request's tokens are the same with and without chained steps (the stand-in's logits depend on the
    context alone), the cache manager's invariants hold after every step, and chains do happen."""
    rng = random.Random(1000 + seed)
    pages = rng.choice([16, 24, 60])
    extra = rng.choice([(), (5, 9)])
    loops = []
    for cls in (PythonLoop, ChainLoop):
        cache, sched = make_scheduler(pages)
        loops.append(cls(sched, cache, extra_stops=extra))
    plain_loop, chain_loop = loops
    arrivals = sorted((rng.choice([0, 0, 0, 6, 20, 21, 50]), [rng.randrange(VOCAB) for _ in range(rng.randint(1, 30))],
                       random_params(random.Random(seed * 77 + i))) for i in range(10))
    cancel_at = {rng.randint(3, 40): rng.randint(1, 10)}
    ids = {}
    for loop in loops:
        now, step, idle = 0, 0, 0
        while step < 400:
            for i, (at, prompt, params) in enumerate(arrivals):
                if at == step:
                    ids.setdefault(i, []).append(loop.add_request(prompt, params, now))
            if step in cancel_at:
                loop.cancel(cancel_at[step])
            events = loop.step(now)
            loop.cache.check_invariants()
            idle = idle + 1 if events is None else 0
            now += 1000
            step += 1
            if idle > 3 and step > 55:
                break
    assert not plain_loop.active and not chain_loop.core.has_unfinished()
    cancelled = set(cancel_at.values())
    for i, (a, b) in ids.items():
        assert a == b
        rec = chain_loop.core.record(b)
        if a in cancelled:             # a cancelled request ends at a moment that depends on the step count
            assert rec.finished and plain_loop.outputs[a]["finished"]
            continue
        assert rec.tokens == plain_loop.outputs[a]["tokens"], f"request {a}"
        assert rec.reason.name == plain_loop.outputs[a]["reason"]
    assert chain_loop.cache.stats(0)["live"] == 0
    assert chain_loop.core.chained_steps == chain_loop.launches.count("ahead")
    test_steps_launched_ahead_change_no_token.chained = getattr(test_steps_launched_ahead_change_no_token, "chained", 0) + chain_loop.core.chained_steps


def test_chains_do_happen_and_end_where_they_must():
    cache, sched = make_scheduler(pages=60, max_batch_seqs=4)
    loop = ChainLoop(sched, cache)
    greedy = rt.SamplingParams(0.0, 1.0, None, 9, 0, [], None, True)
    a = loop.add_request([1, 2, 3, 4, 5], greedy, 0)
    b = loop.add_request([7, 8], rt.SamplingParams(0.8, 1.0, None, 6, 0, [], 11, True), 0)
    now = 0
    while loop.core.has_unfinished():
        loop.step(now)
        cache.check_invariants()
        now += 1000
    # step 0 is the prefill of both; the decodes chain until b nears its limit, then a alone chains until its own
    assert loop.launches[0] == "now" and loop.launches.count("ahead") >= 5
    assert len(loop.core.record(a).tokens) == 9 and len(loop.core.record(b).tokens) == 6
    assert loop.core.dropped_chains == 0
    # a request that needs a ranking on the host, or one that waits for admission, keeps the steps unchained
    cache, sched = make_scheduler(pages=60, max_batch_seqs=4)
    loop = ChainLoop(sched, cache)
    loop.add_request([1, 2, 3], rt.SamplingParams(1.0, 0.9, None, 6, 0, [], None, True), 0)
    now = 0
    while loop.core.has_unfinished():
        loop.step(now)
        now += 1000
    assert loop.launches.count("ahead") == 0
    # a stop token ends a chained request: its row in the step launched ahead is passed over
    cache, sched = make_scheduler(pages=60, max_batch_seqs=4)
    loop = ChainLoop(sched, cache)
    prompt = [9, 9, 9]
    free_run, ctx = [], list(prompt)
    for _ in range(8):
        free_run.append(int(np.argmax(pseudo_logits(ctx))))
        ctx.append(free_run[-1])
    stop_at = free_run[4]
    first = free_run.index(stop_at)
    rid = loop.add_request(prompt, rt.SamplingParams(0.0, 1.0, None, 20, 0, [stop_at], None, True), 0)
    other = loop.add_request([4, 4], rt.SamplingParams(0.0, 1.0, None, 12, 0, [], None, True), 0)
    now = 0
    while loop.core.has_unfinished():
        loop.step(now)
        cache.check_invariants()
        now += 1000
    assert loop.core.record(rid).tokens == free_run[:first] and loop.core.record(rid).reason == rt.FinishReason.Stop
    assert len(loop.core.record(other).tokens) == 12 and loop.launches.count("ahead") >= 3
