"""The engine: scheduler above the step function, sampling below it.

One ``step()`` is what the reference's engine loop does per iteration
(crates/stride-engine/src/lib.rs:299-414): ask the scheduler for a batch, build
the work items (portions first, then decodes; logits where a portion reaches the
end of the context), run the step function, sample one token per returned row,
feed tokens back, stop sequences that drew a stop token (which is not appended)
and retire those that reached their limit. Time is a logical clock in
microseconds advanced by each step's measured duration, or by 1000 when nothing
could be scheduled (lib.rs:301-306,379).

Sampling: greedy and plain-temperature rows are drawn by a kernel on the device
(only token ids come back to the host); rows with top-k or top-p are ranked by
the host sampler from their logits. Either way the request's own seeded
generator supplies the uniform number.
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..config import EngineConfig, config_from_dict
from ..csrc import ops
from ..csrc.build import load_runtime
from .loading import attach_cache, load_model, plan_cache, random_model
from .runner import ModelRunner


_NVTX = os.environ.get("STRIDE_B200_NVTX", "0") == "1"      # named ranges around every step, for a timeline profiler


class EngineBusy(RuntimeError):
    """``add_request`` refuses: too many requests wait for admission already."""


@dataclass
class RequestOutput:
    request_id: int
    prompt_len: int
    tokens: list
    finished: bool = False
    finish_reason: Optional[str] = None
    cached_prompt_tokens: int = 0
    ttft_us: Optional[int] = None
    mean_itl_us: Optional[float] = None
    seed: int = 0


class _Active:
    __slots__ = ("request_id", "seq", "sampler", "greedy", "ranked", "temperature", "output")

    def __init__(self, request_id, seq, sampler, output):
        self.request_id, self.seq, self.sampler, self.output = request_id, seq, sampler, output
        p = sampler.params
        self.greedy = p.is_greedy()
        self.ranked = p.needs_ranking()
        self.temperature = 0.0 if self.greedy else float(p.temperature)


class Engine:
    """``Engine(model_dir)`` loads a checkpoint folder; ``Engine(config=dict_or_typed,
    random_weights=seed)`` builds the architecture with seeded random weights."""

    def __init__(self, model: Optional[str] = None, *, config=None, random_weights: Optional[int] = None,
                 engine_config: Optional[EngineConfig] = None, eos_token_id: Optional[int] = None, device="cuda", **options):
        ops.require_device()
        self.cfg = engine_config or EngineConfig(**options)
        if engine_config is not None and options:
            raise TypeError("give either engine_config or keyword options, not both")
        self._rt = load_runtime()
        token_cap = self.cfg.max_batch_tokens
        row_cap = min(self.cfg.max_batch_seqs, token_cap)
        if model is not None:
            self.model_config, self.model = load_model(model, self.cfg.dtype, device, token_cap, row_cap)
        elif config is not None:
            self.model_config = config_from_dict(config) if isinstance(config, dict) else config
            if random_weights is None:
                raise ValueError("a configuration without a model folder needs random_weights=<seed>")
            self.model = random_model(self.model_config, random_weights, self.cfg.dtype, device, token_cap, row_cap)
        else:
            raise ValueError("give a model folder or a configuration")
        spec = self.model.spec
        self.max_model_len = min(self.cfg.max_model_len, spec.max_positions)
        plan = plan_cache(self.model, self.cfg.block_size, self.cfg.num_blocks, self.cfg.activation_reserve,
                          self.cfg.max_batch_seqs, self.model.rt.dtype)
        self.device_cache, self.cache = attach_cache(self.model, plan, self.cfg.prefix_caching)
        self.runner = ModelRunner(self.model, self.cache, token_capacity=token_cap, seq_capacity=self.cfg.max_batch_seqs,
                                  row_capacity=row_cap, max_model_len=self.max_model_len, cuda_graphs=self.cfg.cuda_graphs)
        self.scheduler = self._rt.Scheduler(
            self._rt.SchedulerConfig(self.cfg.max_batch_seqs, self.cfg.max_batch_tokens, self.max_model_len,
                                     self.cfg.watermark, self.cfg.chunked_prefill), self.cache)
        self.eos = eos_token_id if eos_token_id is not None else (spec.eos_token_ids[0] if spec.eos_token_ids else -1)
        self.extra_eos = tuple(spec.eos_token_ids[1:]) if eos_token_id is None else ()
        self.now = 0
        self._next_request = 1
        self._active: dict[int, _Active] = {}           # by sequence id
        self._outputs: dict[int, RequestOutput] = {}    # by request id
        self._seq_of_request: dict[int, int] = {}
        pin = self.model.rt.device.type == "cuda"
        self._sample_host = torch.zeros(3 * row_cap, dtype=torch.float32, pin_memory=pin)
        self._sample_dev = torch.zeros(3 * row_cap, dtype=torch.float32, device=self.model.rt.device)
        self._tokens_dev = torch.zeros(row_cap, dtype=torch.int32, device=self.model.rt.device)
        self._tokens_host = torch.zeros(row_cap, dtype=torch.int32, pin_memory=pin)
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=pin)     # the kernels' timed-out-wait word, read back with the tokens
        self._row_cap = row_cap
        self.forward_passes = 0
        self.last_step: dict = {}
        self.busy_us = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ---------------------------------------------------------------- requests
    def add_request(self, tokens: Sequence[int], params=None, tenant: str = "default", klass: str = "interactive") -> int:
        """Queues one request; returns its id. Raises ValueError when the
        sampling parameters are invalid, the prompt is empty or too long, or a
        token lies outside the vocabulary."""
        if self.scheduler.num_waiting >= self.cfg.max_queued:
            # the reference's engine tells its API layer to back off at this point (crates/stride-engine/src/lib.rs:68-70)
            raise EngineBusy(f"{self.scheduler.num_waiting} requests are waiting for admission (max_queued {self.cfg.max_queued})")
        params = params if params is not None else self._rt.SamplingParams()
        tokens = [int(t) for t in tokens]
        for t in tokens:
            if not 0 <= t < self.model.vocab:
                raise ValueError(f"token {t} lies outside the vocabulary of {self.model.vocab}")
        if self.extra_eos:
            params = self._with_stops(params, self.extra_eos)
        service = {"interactive": self._rt.ServiceClass.Interactive, "batch": self._rt.ServiceClass.Batch,
                   "background": self._rt.ServiceClass.Background}[klass]
        rid = self._next_request
        seq = self.scheduler.admit(rid, tenant, tokens, params, service, self.now)
        self._next_request += 1
        # fallback seed: base + request id (+ index 0), crates/stride-engine/src/lib.rs:278-287
        seed = (self.cfg.seed + rid) & 0xFFFFFFFFFFFFFFFF
        sampler = self._rt.Sampler(params, self.eos, seed)
        out = RequestOutput(rid, len(tokens), [], seed=sampler.effective_seed)
        self._active[seq] = _Active(rid, seq, sampler, out)
        self._outputs[rid] = out
        self._seq_of_request[rid] = seq
        return rid

    def _with_stops(self, params, extra):
        p = self._rt.SamplingParams(params.temperature, params.top_p, params.top_k, params.max_tokens, params.min_tokens,
                                    list(params.stop_tokens) + [e for e in extra if e not in params.stop_tokens],
                                    params.seed, params.ignore_eos)
        return p

    def cancel(self, request_id: int) -> None:
        for f in self.scheduler.cancel(request_id):
            self._retire(f.seq, "cancelled", f)

    def has_unfinished(self) -> bool:
        return bool(self._active)

    def output(self, request_id: int) -> RequestOutput:
        return self._outputs[request_id]

    # -------------------------------------------------------------------- step
    def step(self) -> list:
        """One scheduling step. Returns [(request_id, token or None, finish_reason or None)]:
        a token for every request that produced one, and a reason for every
        request that ended in this step."""
        batch = self.scheduler.step(self.now)
        if self.cfg.check_invariants:
            self.cache.check_invariants()
        if batch.is_empty():
            self.now += 1000
            return []
        started = time.perf_counter()
        step_batch = self.scheduler.build_batch(batch)
        if _NVTX:
            torch.cuda.nvtx.range_push(f"stride.step tokens={step_batch.num_tokens} seqs={step_batch.num_seqs}")
        logits = self.runner.step(step_batch)
        seqs = step_batch.row_requests()
        tokens = self._sample(logits, seqs)
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        self.scheduler.after_step(batch)
        duration = int((time.perf_counter() - started) * 1e6)
        # the record of the step (python/stride_worker/model.py:238-240,343-345 measures the same span on the worker)
        self.last_step = {"tokens": step_batch.num_tokens, "seqs": step_batch.num_seqs, "rows": len(seqs),
                          "decode_only": step_batch.decode_only, "us": duration}
        self.forward_passes += 1
        self.busy_us += duration
        self.now += max(duration, 1)
        self.h2d_bytes += self.runner.last_h2d_bytes
        events, sampled, stopped = [], [], []
        for seq, token in zip(seqs, tokens):
            a = self._active.get(seq)
            if a is None:
                continue
            if a.sampler.is_stop(token):
                stopped.append(seq)
            else:
                sampled.append((seq, token))
                a.output.tokens.append(token)
                events.append((a.request_id, token, None))
        finished = self.scheduler.on_tokens(sampled, self.now)
        for seq in stopped:
            f = self.scheduler.stop(seq)
            events.append((self._active[seq].request_id, None, "stop"))
            self._retire(seq, "stop", f)
        for f in finished:
            events.append((self._active[f.seq].request_id, None, "length"))
            self._retire(f.seq, "length", f)
        if self.cfg.check_invariants:
            self.cache.check_invariants()
        return events

    def _retire(self, seq, reason, finished) -> None:
        a = self._active.pop(seq, None)
        if a is None:
            return
        a.output.finished = True
        a.output.finish_reason = reason
        if finished is not None:
            a.output.cached_prompt_tokens = finished.cached_prefix_len
            a.output.ttft_us = finished.ttft_us
            a.output.mean_itl_us = finished.mean_itl_us
        self._seq_of_request.pop(a.request_id, None)
        self.scheduler.forget(seq)

    # ---------------------------------------------------------------- sampling
    def _sample(self, logits: torch.Tensor, seqs: list) -> list:
        n = len(seqs)
        if n == 0:
            return []
        cap = self._row_cap
        host = self._sample_host.numpy()
        temperature, uniform = host[:cap], host[cap:2 * cap]
        suppress = host[2 * cap:3 * cap].view(np.int32)
        ranked_rows = []
        for r, seq in enumerate(seqs):
            a = self._active[seq]
            generated = len(a.output.tokens)
            suppress[r] = a.sampler.suppressed_token(generated)
            if a.ranked:
                ranked_rows.append(r)
                temperature[r] = 0.0
                uniform[r] = 0.0
            else:
                temperature[r] = a.temperature
                uniform[r] = 0.0 if a.greedy else a.sampler.next_uniform()
        self._sample_dev.copy_(self._sample_host, non_blocking=True)
        dev = self._sample_dev
        ops.sample_rows(logits, self._tokens_dev[:n], temperature=dev[:n], uniform=dev[cap:cap + n],
                        suppress=dev[2 * cap:2 * cap + n].view(torch.int32))
        self._tokens_host[:n].copy_(self._tokens_dev[:n], non_blocking=True)
        self._status_host.copy_(ops.status_tensor(self._tokens_dev.device)[:1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        ops.raise_on_kernel_status(int(self._status_host[0]))
        self.h2d_bytes += self._sample_host.numel() * 4
        self.d2h_bytes += n * 4 + 4
        tokens = self._tokens_host[:n].tolist()
        if ranked_rows:
            rows = logits[torch.as_tensor(ranked_rows, device=logits.device)].cpu().numpy()
            self.d2h_bytes += rows.nbytes
            for i, r in enumerate(ranked_rows):
                a = self._active[seqs[r]]
                tokens[r] = a.sampler.sample(rows[i], len(a.output.tokens))
        return tokens

    # ------------------------------------------------------------ conveniences
    def generate(self, prompts: Sequence[Sequence[int]], params=None, tenant: str = "default",
                 klass: str = "interactive") -> list:
        """Runs the prompts to completion and returns a ``RequestOutput`` for each,
        in the order given. ``params`` is one SamplingParams for all or a list."""
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        ids = [self.add_request(p, sp, tenant, klass) for p, sp in zip(prompts, plist)]
        idle_steps = 0
        while any(not self._outputs[i].finished for i in ids):
            if self.step():
                idle_steps = 0
            else:
                idle_steps += 1
                if idle_steps > 10000:
                    raise RuntimeError("the scheduler could not place any work for 10000 steps")
        return [self._outputs[i] for i in ids]

    def forward(self, work: Sequence[tuple]) -> torch.Tensor:
        """The raw step function on explicit work: [(request_key, tokens, position, want)].
        The caller manages pages through ``engine.cache`` (open / ensure / close)."""
        batch = self._rt.StepBatch(self.cache)
        for key, tokens, position, want in work:
            batch.add(int(key), [int(t) for t in tokens], int(position), [int(w) for w in want])
        return self.runner.step(batch)

    def get_weight(self, name: str) -> torch.Tensor:
        return self.model.get_weight(name)

    def cache_stats(self, group: int = 0) -> dict:
        return self.cache.stats(group)

    def metrics(self) -> dict:
        """Scheduler, cache and engine counters (crates/stride-engine/src/lib.rs:49-63)."""
        kv = self.cache.stats(0)
        m = dict(self.scheduler.metrics())
        m.update(forward_passes=self.forward_passes, busy_us=self.busy_us, kv_blocks_total=kv["capacity"],
                 kv_blocks_live=kv["live"], kv_blocks_cached=kv["cached"], kv_block_hit_rate=kv["block_hit_rate"],
                 queued=self.scheduler.num_waiting, running=self.scheduler.num_running,
                 graph_replays=self.runner.graph_replays, h2d_bytes=self.h2d_bytes, d2h_bytes=self.d2h_bytes)
        return m
