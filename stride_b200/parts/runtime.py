"""What parts share at run time: the device, the compute dtype, reusable
activation buffers, and the residual stream.

Buffers are allocated once per tag at the step's token capacity and reused by
every layer and every step, so a step allocates nothing and the addresses that
a captured CUDA graph holds stay valid.
"""

from __future__ import annotations

import torch

from ..csrc import ops


class Runtime:
    def __init__(self, device, dtype: torch.dtype, token_capacity: int, row_capacity: int):
        self.device = torch.device(device)
        self.dtype = dtype
        self.token_capacity = int(token_capacity)
        self.row_capacity = int(row_capacity)
        self._buffers: dict[tuple, torch.Tensor] = {}
        self._shared: dict = {}
        self._retired: list = []

    def buffer(self, tag: str, rows: int, cols: int, dtype: torch.dtype | None = None, row_kind: str = "tokens"):
        """A [rows, cols] view of the buffer ``tag``. ``row_kind`` picks the
        capacity: "tokens" (the step's tokens) or "rows" (wanted logit rows)."""
        dtype = dtype or self.dtype
        cap = self.token_capacity if row_kind == "tokens" else self.row_capacity
        if rows > cap:
            raise ValueError(f"buffer {tag!r}: {rows} rows exceed the capacity {cap}")
        key = (tag, cols, dtype, row_kind)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def scratch(self, tag: str, numel: int, dtype: torch.dtype = torch.float32):
        """A flat scratch buffer of at least ``numel`` elements. It only ever grows,
        and growing happens outside graph capture (the warm-up run of a bucket
        asks for the same size as the captured run); a buffer that was outgrown
        stays allocated, because an earlier graph may hold its address. New buffers
        are zeroed: kernels that count themselves off on tickets keep those in
        their scratch, zero between launches."""
        key = ("scratch", tag, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)      # a captured graph may still write to it: never hand it back
            buf = torch.zeros(int(numel), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf

    def shared(self, key, make):
        """One object per key for all parts (e.g. a rotary table shared by all layers)."""
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]

    def buffer_bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class ResidualStream:
    """The residual stream of one step: a float32 [tokens, hidden] tensor plus at
    most one pending delta. ``add`` defers the sum so that the next ``normed``
    can fuse it with the norm (``Norm.apply``): x = residual + delta in float32,
    written back, and norm(x) out, in one kernel for RMSNorm."""

    def __init__(self, runtime: Runtime, tokens: int, hidden: int):
        self.rt = runtime
        self.tokens = tokens
        self.hidden = hidden
        self.residual = runtime.buffer("residual", tokens, hidden, torch.float32)
        self._pending = None

    def add(self, delta) -> None:
        if self._pending is not None:
            ops.add_residual(self.residual, self._pending)
        self._pending = delta

    def normed(self, norm, rows=None, tag: str = "normed"):
        """norm(residual + pending). With ``rows`` (int32 indices) only those rows
        are produced and the residual is left as it is."""
        if rows is None:
            out = self.rt.buffer(tag, self.tokens, self.hidden)
            norm.apply(self.residual, self._pending, out)
            self._pending = None
        else:
            out = self.rt.buffer(tag + "_rows", rows.shape[0], self.hidden, row_kind="rows")
            norm.apply(self.residual, self._pending, out, rows=rows)
        return out

    def materialize(self):
        """The stream with every pending sum applied (float32)."""
        if self._pending is not None:
            ops.add_residual(self.residual, self._pending)
            self._pending = None
        return self.residual
