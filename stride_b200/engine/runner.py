"""The step function: runs one batch of (request, its next tokens) through the
model from the cache and returns the logits at the wanted places.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere
(python/stride_worker/model.py:225-346 is the reference's step). The host packs
the index arrays once, copies them with one transfer from pinned memory and
launches the kernels on the current stream. Decode-only batches are padded to a
bucket size and replayed from a CUDA graph captured for that bucket, which
removes the launch cost of the several hundred kernels of a step.
"""

from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from ..csrc.build import load_runtime
from .context import make_context


def _buckets(limit: int) -> list[int]:
    out, b = [], 1
    while b < limit:
        out.append(b)
        b *= 2
    out.append(limit)
    return out


class _Staging:
    """Pinned host buffer + device buffer of one packed layout."""

    def __init__(self, layout: dict, device):
        self.layout = layout
        pin = torch.device(device).type == "cuda"
        self.host = torch.zeros(layout["total"], dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(layout["total"], dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event() if pin else None

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        if self.copied is not None:
            self.copied.record()

    def wait_host_free(self) -> None:
        if self.copied is not None:
            self.copied.synchronize()


class ModelRunner:
    CONTEXT_BUCKET_BASE = 2048      # the smallest context bound a decode graph is captured for

    def __init__(self, model, cache_manager, *, token_capacity: int, seq_capacity: int, row_capacity: int,
                 max_model_len: int, cuda_graphs: bool = True):
        ops.require_device()
        self.model = model
        self.cache = cache_manager
        self.rt = model.rt
        self.device = self.rt.device
        self.groups = cache_manager.num_groups
        self.token_capacity, self.seq_capacity, self.row_capacity = token_capacity, seq_capacity, row_capacity
        if max_model_len > model.spec.max_positions:
            raise ValueError(f"max_model_len {max_model_len} exceeds the {model.spec.max_positions} positions the model's "
                             "position tables hold")
        self.max_model_len = int(max_model_len)
        self.table_width = max(1, cache_manager.pages_for(max_model_len))
        self._rt_mod = load_runtime()
        self._eager = _Staging(self._rt_mod.packed_layout(self.groups, token_capacity, seq_capacity, row_capacity,
                                                          self.table_width), self.device)
        self.cuda_graphs = cuda_graphs and model.graph_safe
        self._decode_buckets = _buckets(min(seq_capacity, token_capacity))
        self._graphs: dict[tuple, tuple] = {}        # (batch bucket, context bucket) -> (graph, logits)
        self._stagings: dict[int, _Staging] = {}     # batch bucket -> packed step arrays
        self._token_source = None
        self.steps = 0
        self.graph_replays = 0
        self.last_h2d_bytes = 0
        self.launches_per_graph: dict = {}
        self.replayed_launches = 0      # own kernels run through graph replays

    # ------------------------------------------------------------------ public
    def step(self, batch, to_host: bool = False, token_source=None):
        """Runs ``batch`` (a runtime ``StepBatch``). Returns float32 logits
        [batch.num_rows, vocab] in the order of the wanted places: a view of a
        reused device buffer, valid until the next step — or a CPU tensor when
        ``to_host`` is set or the rows exceed the row capacity (they are then
        produced in slices). ``token_source`` (int32 on the device, one per token of
        the batch): the token ids are taken from there instead of from the batch,
        by a copy on the device after the step's arrays have been uploaded; this is
        how a step runs on tokens that the step before it has only just sampled."""
        self._token_source = token_source
        if token_source is not None and token_source.shape[0] != batch.num_tokens:
            raise ValueError("one token id per token of the step is needed")
        self.steps += 1
        if batch.num_tokens == 0:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device="cpu" if to_host else self.device)
        if batch.num_tokens > self.token_capacity or batch.num_seqs > self.seq_capacity:
            raise ValueError(f"the step has {batch.num_tokens} tokens of {batch.num_seqs} requests; the runner was sized "
                             f"for {self.token_capacity} and {self.seq_capacity}")
        # Checked here, on the host, for every caller (scheduler, trace replay, the raw step function): the block
        # table is as wide as max_model_len rounded up to a page, but the position tables end at max_model_len, and
        # no kernel checks a position against them (python/stride_worker/cache.py:82-86 raises before it touches memory).
        if batch.max_ctx > self.max_model_len or batch.max_pages > self.table_width:
            raise ValueError(f"a request would reach position {batch.max_ctx - 1}; max_model_len is {self.max_model_len}")
        if self.cuda_graphs and batch.decode_only and batch.num_rows == batch.num_seqs:
            logits = self._step_graph(batch)
            return logits.cpu() if to_host else logits
        if self.cuda_graphs and batch.num_seqs == 1 and batch.num_tokens == self.token_capacity and batch.num_rows <= 1:
            logits = self._step_full_portion(batch)
            return logits.cpu() if to_host else logits
        return self._step_eager(batch, to_host)

    def timed_step(self, batch):
        """The same step run eagerly with CUDA events around every launch: ``(logits, {class of kernel:
        milliseconds})``. For looking at where a step's time goes; a step that generation runs is not timed."""
        self._token_source = None
        if batch.num_tokens > self.token_capacity or batch.num_seqs > self.seq_capacity or batch.max_ctx > self.max_model_len:
            raise ValueError("the step does not fit the runner")
        with ops.KernelTimer() as timer:
            logits = self._step_eager(batch, to_host=False)
        return logits, timer.milliseconds()

    # ------------------------------------------------------------------- eager
    def _context(self, staging, batch, num_tokens, num_rows, for_graph: int = 0):
        items, row = [], 0
        for request, tokens, position, _want in batch.items():
            items.append((request, row, len(tokens), position, self.cache.state_slot(request)))
            row += len(tokens)
        tail_seq = len(items)
        while tail_seq > 0 and items[tail_seq - 1][2] == 1:
            tail_seq -= 1
        tail_start = items[tail_seq][1] if tail_seq < len(items) else row
        bound = for_graph if for_graph else batch.max_ctx       # a captured graph is sized for its context bucket
        return make_context(staging.dev, staging.layout, num_tokens, batch.num_seqs, num_rows, max_q_len=batch.max_q_len,
                            max_ctx=batch.max_ctx, decode_only=batch.decode_only, host_items=items,
                            decode_tail_start=0 if for_graph else tail_start, decode_tail_seq=0 if for_graph else tail_seq,
                            context_bound=bound)

    def _pack(self, staging, batch):
        l = staging.layout
        staging.wait_host_free()
        batch.pack(self.groups, l["token_cap"], l["seq_cap"], l["row_cap"], l["table_width"], staging.host_np)
        staging.upload()
        source = self._token_source
        if source is not None:
            staging.dev[l["token_ids"]: l["token_ids"] + source.shape[0]].copy_(source)
        self.last_h2d_bytes = l["total"] * 4

    def _step_eager(self, batch, to_host):
        rows = batch.num_rows
        if rows <= self.row_capacity:
            self._pack(self._eager, batch)
            ctx = self._context(self._eager, batch, batch.num_tokens, rows)
            logits = self.model.forward(ctx)
            return logits.cpu() if to_host else logits
        # More rows wanted than the logits buffer holds: run the layers once and
        # the head slice by slice, gathering on the host.
        l = self._eager.layout
        self._eager.wait_host_free()
        all_rows = self._wanted_rows(batch)
        out = torch.empty((rows, self.model.vocab), dtype=torch.float32)
        stream = None
        for lo in range(0, rows, self.row_capacity):
            hi = min(rows, lo + self.row_capacity)
            if stream is None:
                batch.pack(self.groups, l["token_cap"], l["seq_cap"], l["row_cap"], l["table_width"], self._eager.host_np,
                           row_offset=lo, row_count=hi - lo)
                self._eager.upload()
                ctx = self._context(self._eager, batch, batch.num_tokens, hi - lo)
                stream = self.model.forward_layers(ctx)
            else:
                ctx.logit_rows[:hi - lo].copy_(torch.as_tensor(all_rows[lo:hi], dtype=torch.int32), non_blocking=False)
                ctx.num_rows = hi - lo
            out[lo:hi] = self.model.forward_head(stream, ctx).cpu()
        return out

    @staticmethod
    def _wanted_rows(batch):
        rows, at = [], 0
        for _request, tokens, _position, want in batch.items():
            rows.extend(at + w for w in want)
            at += len(tokens)
        return rows

    # ------------------------------------------------------------------ graphs
    def _bucket(self, n: int) -> int:
        for b in self._decode_buckets:
            if b >= n:
                return b
        return self._decode_buckets[-1]

    def _context_bucket(self, max_ctx: int) -> int:
        """The context bound a decode graph is captured for: 2048, 3072, 4096, 5120, 7168, 9216, ... (a quarter
        more each time, in steps of 1024), at most what the block table holds. Kernels size their grids and
        choose their splits from the bound, so a short context does not pay for max_model_len; a growing one
        moves to the next graph every 25 % of its length."""
        full = self.table_width * self.cache.page_size
        step = max(1, self.CONTEXT_BUCKET_BASE // 2)
        bound = self.CONTEXT_BUCKET_BASE
        while bound < max_ctx and bound < full:
            bound = -(-(bound * 5 // 4) // step) * step
        return min(bound, full)

    def _step_graph(self, batch):
        b = self._bucket(batch.num_seqs)
        cb = self._context_bucket(batch.max_ctx)
        staging = self._stagings.get(b)
        if staging is None:
            staging = self._stagings[b] = _Staging(self._rt_mod.packed_layout(self.groups, b, b, b, self.table_width), self.device)
        entry = self._graphs.get((b, cb))
        if entry is None:
            self._pack(staging, batch)
            ctx = self._context(staging, batch, b, b, for_graph=cb)
            self._warm_up(ctx, batch)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.counters["launches"]
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
            self.launches_per_graph[b] = ops.counters["launches"] - before
            entry = (graph, logits)
            self._graphs[(b, cb)] = entry
        graph, logits = entry
        self._pack(staging, batch)
        graph.replay()
        self.graph_replays += 1
        self.replayed_launches += self.launches_per_graph[b]
        return logits[:batch.num_rows]

    def _step_full_portion(self, batch):
        """One request's portion that fills the token budget (every step but the last of a long prompt cut into
        portions, when nothing else is running): always the same launches, whatever the position, so it is
        replayed from a graph too, one for the portions that want no logits and one for those that want a row."""
        key = ("portion", batch.num_rows)
        entry = self._graphs.get(key)
        if entry is None:
            self._pack(self._eager, batch)
            ctx = self._context(self._eager, batch, batch.num_tokens, batch.num_rows)
            self._warm_up(ctx, batch)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.counters["launches"]
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
            self.launches_per_graph[key] = ops.counters["launches"] - before
            entry = (graph, logits)
            self._graphs[key] = entry
        graph, logits = entry
        self._pack(self._eager, batch)
        graph.replay()
        self.graph_replays += 1
        self.replayed_launches += self.launches_per_graph[key]
        return logits[:batch.num_rows]

    def _warm_up(self, ctx, batch) -> None:
        """One eager run before a capture: it allocates every buffer the step touches and loads what is loaded
        lazily. The replay that follows runs the same step again. Writing keys and values twice is harmless (the
        same values to the same places); per-request state is not idempotent, so the rows of the step's requests
        are put back as they were, and the replay is the one run that counts."""
        states = self.model._states()
        if not states:
            self.model.forward(ctx)
            return
        slots = torch.as_tensor([self.cache.state_slot(request) for request, _t, _p, _w in batch.items()], dtype=torch.long,
                                device=self.device)
        kept = [state[slots].clone() for state in states]
        self.model.forward(ctx)
        for state, rows in zip(states, kept):
            state[slots] = rows

    def captured_buckets(self) -> list[int]:
        return sorted({k[0] for k in self._graphs if k[0] != "portion"})
