"""Rotary position encoding with optional llama3 frequency rescaling.

The table is built once per distinct spec, in float32, as the reference builds it
(python/stride_worker/layers.py:38-82): inv_freq = theta^(-2j/hd); with llama3
scaling, wavelengths above original/low are divided by ``factor``, those between
original/high and original/low are interpolated, the rest stay; angle =
position * inv_freq. Only the half table [max_positions, hd/2] is kept, since the
reference's full table repeats it. The rotation itself and the write of keys and
values into pages are one kernel (``rope_kv_write``); angles, products and sums
are float32 in both modes.
"""

from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import PositionEncoding, register_part


def rope_inverse_frequencies(head_dim: int, theta: float, scaling) -> torch.Tensor:
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if scaling is not None and scaling.rope_type == "llama3":
        original = scaling.original_max_position_embeddings
        wavelength = 2 * math.pi / inv_freq
        low_wavelength = original / scaling.low_freq_factor
        high_wavelength = original / scaling.high_freq_factor
        scaled = inv_freq / scaling.factor
        smooth = ((original / wavelength - scaling.low_freq_factor) /
                  (scaling.high_freq_factor - scaling.low_freq_factor)).clamp(0.0, 1.0)
        blended = (1 - smooth) * scaled + smooth * inv_freq
        inv_freq = torch.where(wavelength > low_wavelength, scaled, inv_freq)
        inv_freq = torch.where((wavelength <= low_wavelength) & (wavelength >= high_wavelength), blended, inv_freq)
    return inv_freq


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {spec.head_dim}")
        self.max_positions = int(spec.max_positions)
        self._tables = None

    def _build(self):
        inv_freq = rope_inverse_frequencies(self.spec.head_dim, self.spec.theta, self.spec.scaling)
        angles = torch.outer(torch.arange(self.max_positions, dtype=torch.float32), inv_freq)
        return angles.cos().to(self.rt.device), angles.sin().to(self.rt.device)

    def tables(self):
        """(cos, sin), each float32 [max_positions, head_dim / 2]; one pair per distinct spec."""
        if self._tables is None:
            self._tables = self.rt.shared(("rope", self.spec), self._build)
        return self._tables

    def rotation_tables(self):
        cos, sin = self.tables()
        return cos, sin, True

    def encode_and_store(self, qkv, bias, ctx, cache, num_heads, num_kv_heads, head_dim):
        cos, sin = self.tables()
        ops.rope_kv_write(qkv, bias, ctx.positions[:qkv.shape[0]],
                          ctx.slot_mapping[cache.group][:qkv.shape[0]] if cache.writes else None,
                          cos, sin, cache.k_pages, cache.v_pages, num_heads, num_kv_heads, head_dim,
                          cache.page_size, rotate=True)


class NoPositionEncoding(PositionEncoding):
    """Keys and queries stay as they are; keys and values are still stored."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.max_positions = int(spec.max_positions) if spec.max_positions else 1
        self._dummy = runtime.shared(("rope-dummy",), lambda: torch.zeros(8, dtype=torch.float32, device=runtime.device))

    def rotation_tables(self):
        return self._dummy, self._dummy, False

    def encode_and_store(self, qkv, bias, ctx, cache, num_heads, num_kv_heads, head_dim):
        ops.rope_kv_write(qkv, bias, ctx.positions[:qkv.shape[0]],
                          ctx.slot_mapping[cache.group][:qkv.shape[0]] if cache.writes else None,
                          self._dummy, self._dummy, cache.k_pages, cache.v_pages, num_heads, num_kv_heads, head_dim,
                          cache.page_size, rotate=False)


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
