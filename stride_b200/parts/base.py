"""Interfaces of the parts a layer is put together from, and their registry.

A part is built from its spec record and a ``Runtime``; it declares the
checkpoint tensors it reads (``declare``), receives them (``bind``) and runs
(``forward``). Parts know sizes and constants only through their spec.

Interfaces
----------
Norm          ``weight`` (float32 [width]) and ``eps``; applied through
              ``ResidualStream.normed`` so that the preceding residual sum is fused.
Mixer         ``forward(x, ctx, cache) -> delta``: x is the normed input
              [tokens, hidden]; ``cache`` is the ``LayerCache`` of this run. It may
              ask for pages (``cache_request``) and for per-request state of fixed
              size (``state_request``).
FeedForward   ``forward(x, ctx) -> delta``.
PositionEncoding  used by a mixer: ``encode_and_store`` rotates queries and keys
              in place and writes keys and values into the pages.
Layer         ``forward(stream, ctx, cache)``: the arrangement of the above.
Embedding     ``forward(ctx, out)``: fills the float32 residual rows [tokens, hidden]
              from ``ctx.token_ids``; ``table()`` is what a tied head may share.
Head          ``forward(x, out)``: float32 logits [rows, vocab] from the normed rows;
              ``bind(weights, tied)`` receives the embedding's table when its spec
              names no tensor of its own.

Adding a kind: subclass the interface, then ``register_part(category, kind, cls)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..weights import TensorDecl

CATEGORIES = ("norm", "mixer", "feed_forward", "position", "layer", "embedding", "head")
_PARTS: dict[str, dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    _PARTS[category][kind] = cls


def build_part(category: str, spec, runtime):
    try:
        cls = _PARTS[category][spec.kind]
    except KeyError:
        raise ValueError(f"no {category} of kind {spec.kind!r} is registered; known: {sorted(_PARTS[category])}") from None
    return cls(spec, runtime)


def registered_parts(category: str) -> list[str]:
    return sorted(_PARTS[category])


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer keeps per token in pages.

    The plain form is keys and values of one shape: ``CacheRequest(num_kv_heads, head_dim, window)``. A mixer
    that keeps something else names its tensors: ``CacheRequest(tensors=(("latent", 1, 24),))`` keeps one vector
    of 24 numbers per token; ``(("k", 4, 64), ("v", 4, 32))`` keys and values of different widths. Every tensor
    of a request is laid out [num_pages, heads, page_size, width] in the compute dtype and shares the request's
    page ids, so one block table and one slot mapping serve them all.
    """
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None     # None: every token is kept
    tensors: tuple = ()              # of (name, heads, width); empty: ("k", ...) and ("v", ...) of the plain form

    def layout(self) -> tuple:
        if self.tensors:
            return tuple((str(n), int(h), int(w)) for n, h, w in self.tensors)
        return (("k", int(self.num_kv_heads), int(self.head_dim)), ("v", int(self.num_kv_heads), int(self.head_dim)))

    def elements_per_token(self) -> int:
        return sum(h * w for _n, h, w in self.layout())


@dataclass(frozen=True)
class StateRequest:
    """Per-request state of fixed size: one tensor of ``shape`` per live request."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Part:
    # False for a part that reads ``ctx.host_items`` (or otherwise depends on the
    # host's view of a step): such a step is never replayed from a CUDA graph.
    graph_safe = True

    def __init__(self, spec, runtime):
        self.spec = spec
        self.rt = runtime

    def declare(self) -> dict:
        """Checkpoint name -> TensorDecl of every tensor this part reads."""
        return {}

    def bind(self, weights: dict) -> None:
        """Receives the loaded tensors (a dict that holds at least the declared names)."""

    def named_tensors(self) -> dict:
        """Checkpoint name -> device tensor (or a view of a fused one), for inspection."""
        return {}


class Projection:
    """A part's last matrix product, not yet run: ``x @ weight.T``. A mixer or feed-forward that sets
    ``lazy_output`` may return one instead of a tensor when it is called with ``lazy_output=True``; the residual
    stream then runs the product together with the sum and the norm that follow it, or plainly if it cannot."""

    def __init__(self, x, weight):
        self.x, self.weight = x, weight


class Norm(Part):
    def fold_inputs(self):
        """Optional. ``(weight, eps)`` if the norm is ``x * rsqrt(mean(x^2) + eps) * weight`` with a float32
        weight: the residual stream may then fold it into the products before and after it."""
        return None

    def apply(self, residual, pending, out, rows=None) -> None:
        """``x = residual + pending`` in float32 (``pending`` may be None), ``out = norm(x)``. Without ``rows``
        every row is produced and x is written back into ``residual`` (float32 [tokens, hidden]); with ``rows``
        (int32 indices) only those rows are produced, into ``out[i]``, and ``residual`` stays as it is."""
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv, bias, ctx, cache, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError

    def rotation_tables(self):
        """Optional. ``(cos, sin, rotate)`` if what ``encode_and_store`` does is the pairwise rotation of
        ``ops.rope_kv_write`` with these float32 tables (``rotate`` False: no rotation, only the store); a
        mixer may then fold it into its projection. ``None`` (the default): call ``encode_and_store``."""
        return None


class Mixer(Part):
    # True: ``forward`` takes ``lazy_output=True`` and may then return a Projection (its output product, not yet run).
    lazy_output = False
    # True: ``forward`` may be given an ``ops.FoldedNorm`` instead of a normed tensor (``.tensor()`` turns it into one).
    accepts_folded = False

    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    lazy_output = False       # as for Mixer
    accepts_folded = False

    def forward(self, x, ctx):
        raise NotImplementedError


class Layer(Part):
    mixer: Mixer

    def forward(self, stream, ctx, cache) -> None:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx, out) -> None:
        """``out`` (float32 [tokens, hidden], the residual stream) from ``ctx.token_ids[:tokens]``; rows whose
        ``ctx.seq_of_token`` is -1 are padding."""
        raise NotImplementedError

    def table(self):
        """The [vocab, hidden] matrix that a head without a tensor of its own multiplies by, or None."""
        return None


class Head(Part):
    def bind(self, weights: dict, tied=None) -> None:
        """``tied``: the embedding's ``table()`` when the head's spec names no tensor."""

    def forward(self, x, out) -> None:
        """``out`` (float32 [rows, vocab]) from the normed rows ``x`` [rows, hidden]."""
        raise NotImplementedError


__all__ = ["CATEGORIES", "Embedding", "Head", "register_part", "build_part", "registered_parts", "CacheRequest", "StateRequest", "Part", "Norm",
           "PositionEncoding", "Mixer", "FeedForward", "Layer", "TensorDecl", "Projection"]
