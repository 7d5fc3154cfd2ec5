"""The engine: scheduler above the step function, sampling below it.

One ``step()`` is what the reference's engine loop does per iteration
(crates/stride-engine/src/lib.rs:299-414): ask the scheduler for a batch, build
the work items (portions first, then decodes; logits where a portion reaches the
end of the context), run the step function, sample one token per returned row,
feed tokens back, stop sequences that drew a stop token (which is not appended)
and retire those that reached their limit. Time is a logical clock in
microseconds advanced by each step's measured duration, or by 1000 when nothing
could be scheduled (lib.rs:301-306,379).

Every rule of that loop lives in the C++ ``EngineCore`` (``csrc/runtime/
engine_core.hpp``): scheduling, the sampler's parameters, stop rules, retiring.
This class is the device half: it launches the step function and the sampling
kernel between the core's ``begin_step`` and ``finish_step`` and moves the few
bytes in between. When the open step holds single decoded tokens only, the step
after it is launched before this one's tokens are read (``chain_step``): its
token ids are copied on the device from the sampled tokens, so the GPU never
waits for the host between two decode steps.

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


class _Launch:
    """Pinned host buffers of one launched step: the sampler's parameters going in, tokens and the kernels'
    status word coming out. Two of them take turns, since a step may be launched while the one before it is
    still being read."""

    def __init__(self, rows: int, device):
        pin = torch.device(device).type == "cuda"
        self.sample_host = torch.zeros(5 * rows, dtype=torch.float32, pin_memory=pin)
        host = self.sample_host.numpy()
        self.temperature, self.uniform = host[:rows], host[rows:2 * rows]
        self.suppress = host[2 * rows:3 * rows].view(np.int32)
        self.top_k, self.top_p = host[3 * rows:4 * rows].view(np.int32), host[4 * rows:5 * rows]      # 0 and 1: no cut
        self.tokens_host = torch.zeros(rows, dtype=torch.int32, pin_memory=pin)
        self.status_host = torch.zeros(1, dtype=torch.int32, pin_memory=pin)
        self.done = torch.cuda.Event()
        self.rows = 0
        self.ranked: list = []
        self.logits = None
        self.record: dict = {}


_REASONS = {"Length": "length", "Stop": "stop", "Cancelled": "cancelled", "Preempted": "preempted"}


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
        self.core = self._rt.EngineCore(self.scheduler, self.eos, list(self.extra_eos), self.cfg.seed & 0xFFFFFFFFFFFFFFFF,
                                        self.cfg.max_queued, self.model.vocab)
        self.core.set_device_ranks(self.cfg.device_ranking)
        self.now = 0
        self._outputs: dict[int, RequestOutput] = {}    # by request id
        self._seq_of_request: dict[int, int] = {}
        dev = self.model.rt.device
        self._sample_dev = torch.zeros(5 * row_cap, dtype=torch.float32, device=dev)
        self._tokens_dev = torch.zeros(row_cap, dtype=torch.int32, device=dev)
        self._launches = [_Launch(row_cap, dev), _Launch(row_cap, dev)]
        self._turn = 0
        self._ahead: Optional[_Launch] = None           # a step launched before the one before it was read
        self._row_cap = row_cap
        self._mark = None                               # when the device was last known to be busy with a launched step
        self.forward_passes = 0
        self.last_step: dict = {}
        self.busy_us = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ---------------------------------------------------------------- requests
    def add_request(self, tokens: Sequence[int], params=None, tenant: str = "default", klass: str = "interactive") -> int:
        """Queues one request; returns its id. Raises ValueError when the
        sampling parameters are invalid, the prompt is empty or too long, or a
        token lies outside the vocabulary; ``EngineBusy`` when too many requests
        wait for admission already (the reference's engine tells its API layer to
        back off at that point, crates/stride-engine/src/lib.rs:68-70)."""
        params = params if params is not None else self._rt.SamplingParams()
        service = {"interactive": self._rt.ServiceClass.Interactive, "batch": self._rt.ServiceClass.Batch,
                   "background": self._rt.ServiceClass.Background}[klass]
        try:
            rid = self.core.add_request([int(t) for t in tokens], params, tenant, service, self.now)
        except self._rt.EngineBusy as e:
            raise EngineBusy(str(e)) from None
        record = self.core.record(rid)
        self._outputs[rid] = RequestOutput(rid, record.prompt_len, [], seed=record.seed)
        self._seq_of_request[rid] = record.seq
        return rid

    def cancel(self, request_id: int) -> None:
        self._apply(self.core.cancel(request_id))

    def has_unfinished(self) -> bool:
        return self.core.has_unfinished()

    def output(self, request_id: int) -> RequestOutput:
        return self._outputs[request_id]

    # -------------------------------------------------------------------- step
    def step(self) -> list:
        """One scheduling step. Returns [(request_id, token or None, finish_reason or None)]:
        a token for every request that produced one, and a reason for every
        request that ended in this step."""
        core = self.core
        if not core.begin_step(self.now):
            self._ahead = None
            if self.cfg.check_invariants:
                self.cache.check_invariants()
            self.now += 1000
            return []
        if self.cfg.check_invariants:
            self.cache.check_invariants()
        started = time.perf_counter()
        if core.launched_ahead():
            launch = self._ahead
            started = self._mark or started
        else:
            self._ahead = None                  # a chained step that no request survived to use: its results are never read
            launch = self._launch(core.batch(), None)
        self._ahead = None
        try:
            if self.cfg.chain_steps and core.chain_step():
                self._ahead = self._launch(core.next_batch(), launch)
            tokens, ranked_logits = self._collect(launch)
        except ops.KernelError:
            self._fail()
            raise
        self._mark = time.perf_counter()
        duration = int((self._mark - started) * 1e6)
        # the record of the step (python/stride_worker/model.py:238-240,343-345 measures the same span on the worker)
        self.last_step = dict(launch.record, us=duration)
        self.forward_passes += 1
        self.busy_us += duration
        self.now += max(duration, 1)
        events = self._apply(core.finish_step(tokens, launch.ranked, ranked_logits, self.now))
        if self.cfg.check_invariants:
            self.cache.check_invariants()
        return events

    def _launch(self, batch, after: Optional[_Launch]) -> _Launch:
        """Launches the step function and the sampling kernel for ``batch`` and the copies that bring tokens and
        status back; returns without waiting. ``after``: the launch whose sampled tokens are this step's token
        ids (a chained step), copied on the device."""
        launch = self._launches[self._turn]
        self._turn ^= 1
        chained = after is not None
        n = batch.num_rows
        if _NVTX:
            torch.cuda.nvtx.range_push(f"stride.step tokens={batch.num_tokens} seqs={batch.num_seqs} chained={chained}")
        logits = self.runner.step(batch, token_source=self._tokens_dev[:after.rows] if chained else None)
        cap = self._row_cap
        cuts = (launch.top_k, launch.top_p) if self.cfg.device_ranking else (None, None)
        if chained:
            self.core.prepare_next_sampling(launch.temperature, launch.uniform, launch.suppress, *cuts)
            launch.ranked = []
        else:
            launch.ranked = list(self.core.prepare_sampling(launch.temperature, launch.uniform, launch.suppress, *cuts))
        launch.rows, launch.logits = n, logits
        launch.record = {"tokens": batch.num_tokens, "seqs": batch.num_seqs, "rows": n, "decode_only": batch.decode_only,
                         "chained": chained}
        if n:
            dev = self._sample_dev
            dev.copy_(launch.sample_host, non_blocking=True)
            suppress = dev[2 * cap:2 * cap + n].view(torch.int32)
            ops.sample_rows(logits, self._tokens_dev[:n], temperature=dev[:n], uniform=dev[cap:cap + n], suppress=suppress)
            if self.cfg.device_ranking and ((launch.top_k[:n] > 0).any() or (launch.top_p[:n] < 1.0).any()):
                # the rows with a top-k or nucleus cut, over what sample_rows wrote for them
                ops.sample_ranked(logits, self._tokens_dev[:n], dev[:n], dev[cap:cap + n], suppress,
                                  dev[3 * cap:3 * cap + n].view(torch.int32), dev[4 * cap:4 * cap + n])
            launch.tokens_host[:n].copy_(self._tokens_dev[:n], non_blocking=True)
            self.h2d_bytes += launch.sample_host.numel() * 4
        launch.status_host.copy_(ops.status_tensor(self._tokens_dev.device)[:1], non_blocking=True)
        launch.done.record()
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        self.h2d_bytes += self.runner.last_h2d_bytes
        self.d2h_bytes += n * 4 + 4
        return launch

    def _collect(self, launch: _Launch):
        """Waits for one launch (not for what was launched after it) and returns its tokens and, for the rows
        that the host ranks, their logits."""
        launch.done.synchronize()
        ops.raise_on_kernel_status(int(launch.status_host[0]), self._tokens_dev.device)
        tokens = launch.tokens_host[:launch.rows].numpy().copy()
        ranked_logits = None
        if launch.ranked:
            ranked_logits = launch.logits[torch.as_tensor(launch.ranked, device=launch.logits.device)].cpu().numpy()
            self.d2h_bytes += ranked_logits.nbytes
        return tokens, ranked_logits

    def _fail(self) -> None:
        """A kernel reported a failure: the results of the open step (and of a step chained after it) are not to
        be trusted. Their requests end with the reason "error" and give their pages back; the engine goes on with
        the others (python/stride_worker/worker.py:156-165 reports the failed pass and keeps serving)."""
        torch.cuda.synchronize()
        ops.reset_kernel_status(self._tokens_dev.device)
        self._ahead = None
        for rid in self.core.abandon_step():
            self._apply(self.core.cancel(rid, publish=False), reason="error")       # what their pages hold is not to be shared

    def _apply(self, core_events, reason: Optional[str] = None) -> list:
        """Core events into the outputs; returns them as (request, token, reason) tuples."""
        events = []
        for e in core_events:
            out = self._outputs.get(e.request)
            why = None if e.reason == self._rt.FinishReason.NotFinished else (reason or _REASONS[e.reason.name])
            if out is not None:
                if e.token is not None:
                    out.tokens.append(e.token)
                if why is not None:
                    record = self.core.record(e.request)
                    out.finished, out.finish_reason = True, why
                    out.cached_prompt_tokens = record.cached_prefix_len
                    out.ttft_us, out.mean_itl_us = record.ttft_us, record.mean_itl_us
                    self.core.forget(e.request)
                    self._seq_of_request.pop(e.request, None)
            events.append((e.request, e.token, why))
        return events

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
        if self._ahead is not None:
            raise RuntimeError("a step of the engine's own requests is in flight; call step() until they are done")
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
                 graph_replays=self.runner.graph_replays, h2d_bytes=self.h2d_bytes, d2h_bytes=self.d2h_bytes,
                 chained_steps=self.core.chained_steps, dropped_chains=self.core.dropped_chains)
        return m
