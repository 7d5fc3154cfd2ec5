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

Adding a kind: subclass the interface, then ``register_part(category, kind, cls)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..weights import TensorDecl

CATEGORIES = ("norm", "mixer", "feed_forward", "position", "layer")
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
    """Keys and values per token that a mixer keeps in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every key is kept


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


__all__ = ["CATEGORIES", "register_part", "build_part", "registered_parts", "CacheRequest", "StateRequest", "Part", "Norm",
           "PositionEncoding", "Mixer", "FeedForward", "Layer", "TensorDecl", "Projection"]
