"""A decoder put together from a ``ModelSpec``: embedding, layers run in the
order that the spec's schedule gives, final norm, output head.

The schedule is data: an entry names a layer and a cache slot, so a layer may
run twice (with two slots, or sharing one) and a run may read the keys and
values that another run wrote. The step itself follows
python/stride_worker/model.py:225-346: embedding gather, the layers, the final
norm on the wanted rows only, and the head on those rows, giving float32 logits.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import TensorDecl, load_weights
from .base import build_part
from .runtime import ResidualStream, Runtime


class DecoderModel:
    def __init__(self, spec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.layers = [build_part("layer", ls, runtime) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.schedule = tuple(spec.schedule)
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"the schedule names layer {e.layer}, but there are {len(self.layers)} layers")
        self.embed = self.head = None
        self.caches = None          # list of LayerCache, one per schedule entry; set by DeviceCache.attach
        self.capture = None         # when a list, every run appends the float32 hidden state (diagnostics)

    # ----------------------------------------------------------------- weights
    def declare(self) -> dict:
        d = {self.spec.embed_name: TensorDecl((self.vocab, self.hidden))}
        if self.spec.head_name is not None:
            d[self.spec.head_name] = TensorDecl((self.vocab, self.hidden))
        for layer in self.layers:
            d.update(layer.declare())
        d.update(self.final_norm.declare())
        return d

    def load(self, source) -> None:
        """Reads every declared tensor from ``source`` (checked first; one error
        lists all that is missing, unexpected or mis-shaped) and hands them out."""
        weights = load_weights(source, self.declare(), self.rt.dtype, self.rt.device, self.spec.ignorable_tensors)
        self.embed = weights[self.spec.embed_name]
        self.head = weights[self.spec.head_name] if self.spec.head_name is not None else self.embed
        for layer in self.layers:
            layer.bind(weights)
        self.final_norm.bind(weights)

    def named_tensors(self) -> dict:
        d = {self.spec.embed_name: self.embed}
        if self.spec.head_name is not None:
            d[self.spec.head_name] = self.head
        for layer in self.layers:
            d.update(layer.named_tensors())
        d.update(self.final_norm.named_tensors())
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
        ops.embed_gather(ctx.token_ids[:tokens], ctx.seq_of_token[:tokens], self.embed, stream.residual)
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
            ops.linear(normed, self.head, logits)
        return logits

    @property
    def graph_safe(self) -> bool:
        """False when a part needs the host's view of the step and therefore cannot
        be replayed from a captured graph."""
        return all(getattr(p, "graph_safe", True) for layer in self.layers for p in getattr(layer, "parts", lambda: ())())
