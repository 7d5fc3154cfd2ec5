"""Trace replay: feeds given token ids through the model step by step and
returns logits. It samples nothing and schedules nothing; it drives the same
model, step function, cache manager and kernels that generation uses.

A step is ``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}``:
for each request its next tokens and the places among them whose logits are
wanted; all entries of a step run as one batch. Requests listed under ``end``
give their pages back after the step.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from ..csrc.build import load_runtime
from .loading import CachePlan, attach_cache, load_model
from .runner import ModelRunner


class TraceError(ValueError):
    pass


class TraceSession:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", max_tokens: int = 4096, block_size: int = 16,
                 max_requests: int = 8, device="cuda", cuda_graphs: bool = True, model=None, config=None):
        if max_tokens <= 0:
            raise TraceError("--max-tokens must be positive")
        self.block_size = block_size
        capacity = -(-max_tokens // block_size) * block_size
        if model is None:
            # A trace feeds given tokens: it may run past the length that the checkpoint names, as far as the pool reaches.
            config, model = load_model(model_dir, dtype, device, token_capacity=capacity, row_capacity=min(capacity, 256),
                                       min_positions=capacity)
        self.config, self.model = config, model
        plan = CachePlan(block_size, capacity // block_size, max_requests)
        self.device_cache, self.cache = attach_cache(model, plan, prefix_caching=False)
        max_len = min(capacity, model.spec.max_positions)
        self.runner = ModelRunner(model, self.cache, token_capacity=capacity, seq_capacity=max_requests,
                                  row_capacity=model.rt.row_capacity, max_model_len=max_len, cuda_graphs=cuda_graphs)
        self._rt = load_runtime()
        self._keys: dict[str, int] = {}
        self._held: dict[str, int] = {}       # tokens each live request holds
        self._next_key = 1

    def run_step(self, step: dict):
        """Returns float32 logits [wanted, vocab] on the CPU, or None when the
        step wants none."""
        batch = self._rt.StepBatch(self.cache)
        entries = step.get("entries", [])
        seen = set()
        for e in entries:
            rid = str(e["id"])
            tokens = [int(t) for t in e["tokens"]]
            want = [int(w) for w in e.get("want", [])]
            if rid in seen:
                raise TraceError(f"request {rid!r} appears twice in step {step.get('step')}")
            seen.add(rid)
            if not tokens:
                if want:
                    raise TraceError(f"request {rid!r} wants logits but brings no tokens")
                continue
            for t in tokens:
                if not 0 <= t < self.model.vocab:
                    raise TraceError(f"token {t} of request {rid!r} lies outside the vocabulary of {self.model.vocab}")
            if rid not in self._keys:
                self._keys[rid] = self._next_key
                self._next_key += 1
                try:
                    self.cache.open(self._keys[rid], rid)
                except self._rt.OutOfPages:
                    del self._keys[rid]
                    raise TraceError(f"more than {self.cache.slot_capacity} requests are live") from None
                self._held[rid] = 0
            key, position = self._keys[rid], self._held[rid]
            if position + len(tokens) > self.model.spec.max_positions:
                raise TraceError(f"request {rid!r} would pass max_position_embeddings {self.model.spec.max_positions}")
            if not self.cache.ensure(key, position + len(tokens), 0):
                raise TraceError(f"out of cache pages at step {step.get('step')}: request {rid!r} needs "
                                 f"{self.cache.pages_missing(key, position + len(tokens))} more, "
                                 f"{self.cache.num_allocatable} are free (--max-tokens too small for the live requests)")
            batch.add(key, tokens, position, want)
        logits = None
        if batch.num_tokens:
            out = self.runner.step(batch, to_host=True)
            ops.check_kernel_status()
            logits = out if batch.num_rows else None
            for e in entries:
                rid = str(e["id"])
                if e["tokens"]:
                    self._held[rid] += len(e["tokens"])
                    self.cache.trim(self._keys[rid], self._held[rid])
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in self._keys:
                self.cache.close(self._keys.pop(rid))
                del self._held[rid]
        self.cache.check_invariants()
        return logits
