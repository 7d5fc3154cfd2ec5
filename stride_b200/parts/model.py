"""A decoder put together from a ``ModelSpec``: embedding, layers run in the
order that the spec's schedule gives, final norm, output head; each of them a
part chosen by its spec's kind.

The schedule is data: an entry names a layer and a cache slot, so a layer may
run twice (with two slots, or sharing one) and a run may read the keys and
values that another run wrote. The step itself follows
python/stride_worker/model.py:225-346: embedding gather, the layers, the final
norm on the wanted rows only, and the head on those rows, giving float32 logits.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import check_source, load_weights
from .base import build_part
from .runtime import ResidualStream, Runtime


class DecoderModel:
    def __init__(self, spec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.embedding = build_part("embedding", spec.embedding_spec(), runtime)
        self.layers = [build_part("layer", ls, runtime) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.head_spec(), runtime)
        self.schedule = tuple(spec.schedule)
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"the schedule names layer {e.layer}, but there are {len(self.layers)} layers")
        self.caches = None          # list of LayerCache, one per schedule entry; set by DeviceCache.attach
        self.capture = None         # when a list, every run appends the float32 hidden state (diagnostics)

    # ----------------------------------------------------------------- weights
    def _parts(self):
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def declare(self) -> dict:
        d = {}
        for part in self._parts():
            d.update(part.declare())
        return d

    def load(self, source) -> None:
        """Reads every declared tensor from ``source`` (checked first; one error
        lists all that is missing, unexpected or mis-shaped) and hands them out."""
        check_source(source, self.declare(), self.spec.ignorable_tensors)
        # Part by part: a part that fuses tensors at load (q/k/v into one matrix, gate and up interleaved) holds its
        # own copy, so the tensors as stored are dropped as soon as the part has bound them. Loaded all at once, a
        # model whose weights fill most of the device would need them twice.
        for part in self._parts():
            weights = load_weights(source, part.declare(), self.rt.dtype, self.rt.device, checked=True)
            if part is self.head:
                part.bind(weights, tied=self.embedding.table())
            else:
                part.bind(weights)
            del weights

    def named_tensors(self) -> dict:
        d = {}
        for part in self._parts():
            d.update(part.named_tensors())
        return d

    def get_weight(self, name: str) -> torch.Tensor:
        return self.named_tensors()[name]

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self.named_tensors().values():
            key = (t.untyped_storage().data_ptr(), t.storage_offset(), t.numel())
            if key not in seen:
                seen.add(key)
                total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------- cache
    def cache_requests(self):
        """Per cache slot: (CacheRequest or None, StateRequest or None)."""
        slots = {}
        for e in self.schedule:
            mixer = self.layers[e.layer].mixer
            req = (mixer.cache_request(), mixer.state_request())
            if e.cache in slots and slots[e.cache] != req:
                raise ValueError(f"cache slot {e.cache} is shared by mixers with different needs")
            slots[e.cache] = req
        return [slots.get(i, (None, None)) for i in range(self.spec.num_cache_slots)]

    # -------------------------------------------------------------------- step
    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of ``ctx`` and returns float32 logits [rows, vocab]
        for ``ctx.logit_rows`` (a view of a reused buffer)."""
        return self.forward_head(self.forward_layers(ctx), ctx)

    def forward_layers(self, ctx) -> ResidualStream:
        if self.caches is None:
            raise RuntimeError("the model has no cache attached")
        tokens = ctx.num_tokens
        stream = ResidualStream(self.rt, tokens, self.hidden)
        self.embedding.forward(ctx, stream.residual)
        for state in self._states():        # a request that starts in this step finds its state slots at zero
            ops.zero_fresh_state(state, ctx.state_slot, ctx.q_start, ctx.q_len, ctx.positions)
        for entry, cache in zip(self.schedule, self.caches):
            self.layers[entry.layer].forward(stream, ctx, cache)
            if self.capture is not None:
                self.capture.append(stream.materialize().clone())
        return stream

    def forward_head(self, stream: ResidualStream, ctx) -> torch.Tensor:
        """Final norm and output head on ``ctx.logit_rows[:ctx.num_rows]``; may be
        called again with other rows for the same stream."""
        rows = ctx.num_rows
        logits = self.rt.buffer("logits", rows, self.vocab, torch.float32, row_kind="rows")
        if rows:
            normed = stream.normed(self.final_norm, rows=ctx.logit_rows[:rows])
            self.head.forward(normed, logits)
        return logits

    def _states(self) -> list:
        """The per-request state tensors of the attached cache, each once."""
        seen, out = set(), []
        for cache in self.caches or ():
            if cache.state is not None and id(cache.state) not in seen:
                seen.add(id(cache.state))
                out.append(cache.state)
        return out

    @property
    def graph_safe(self) -> bool:
        """False when a part needs the host's view of the step and therefore cannot
        be replayed from a captured graph."""
        return all(getattr(p, "graph_safe", True) for layer in self.layers for p in getattr(layer, "parts", lambda: ())())
