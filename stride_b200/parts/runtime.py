"""What parts share at run time: the device, the compute dtype, reusable
activation buffers, and the residual stream.

Buffers are allocated once per tag at the step's token capacity and reused by
every layer and every step, so a step allocates nothing and the addresses that
a captured CUDA graph holds stay valid.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import Projection


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
        """``delta``: a tensor, or a ``Projection`` (a product not yet run) that the next ``normed`` may fold."""
        self._settle()
        self._pending = delta

    def _settle(self) -> None:
        """Applies what is pending to the residual."""
        if self._pending is not None:
            p = self._pending
            if not (isinstance(p, Projection) and p.weight.shape[0] == self.hidden and ops.rows_wanted(self.tokens)
                    and ops.linear_rows_add(p.x, p.weight, self.residual)):
                ops.add_residual(self.residual, self._run(p))
            self._pending = None

    def _run(self, pending):
        """The pending delta as a tensor (runs a deferred product)."""
        if isinstance(pending, Projection):
            out = self.rt.buffer("projection_out", self.tokens, pending.weight.shape[0])
            ops.linear(pending.x, pending.weight, out)
            return out
        return pending

    def normed(self, norm, rows=None, tag: str = "normed", fold_ok: bool = False):
        """norm(residual + pending). With ``rows`` (int32 indices) only those rows
        are produced and the residual is left as it is. With ``fold_ok`` the caller
        takes an ``ops.FoldedNorm`` too: when the pending delta is a deferred product
        and the norm allows it, product, sum and the norm's statistics become one
        kernel and the norm's scaling is left to the consumer."""
        if rows is None and fold_ok and isinstance(self._pending, Projection):
            folded = self._fold(norm, tag)
            if folded is not None:
                return folded
        if rows is None and isinstance(self._pending, Projection) and self._pending.weight.shape[0] == self.hidden and \
                ops.rows_wanted(self.tokens) and ops.linear_rows_add(self._pending.x, self._pending.weight, self.residual):
            self._pending = None        # the tokens-as-rows product added itself to the residual stream
        pending = None if self._pending is None else self._run(self._pending)
        if rows is None:
            out = self.rt.buffer(tag, self.tokens, self.hidden)
            norm.apply(self.residual, pending, out)
            self._pending = None
        else:
            self._pending = pending
            out = self.rt.buffer(tag + "_rows", rows.shape[0], self.hidden, row_kind="rows")
            norm.apply(self.residual, pending, out, rows=rows)
        return out

    def _fold(self, norm, tag):
        inputs = norm.fold_inputs()
        if inputs is None:
            return None
        weight, eps = inputs
        p = self._pending
        if p.weight.shape[0] != self.hidden:
            return None
        xt = self.rt.buffer(tag + "_folded", self.tokens, self.hidden)
        partials = self.rt.scratch("norm_partials", max(16 * 1024, self.hidden // 32 * ops.ROWS_FOLD_STRIDE))
        stride = 16
        count = ops.linear_add_norm(p.x, p.weight, self.residual, weight, xt, partials)
        if not count and ops.rows_wanted(self.tokens):
            count, stride = ops.linear_rows_add_norm(p.x, p.weight, self.residual, weight, xt, partials), ops.ROWS_FOLD_STRIDE
        if not count:
            return None
        self._pending = None
        return ops.FoldedNorm(xt, partials, count, eps, lambda: self.rt.buffer(tag, self.tokens, self.hidden), stride)

    def materialize(self):
        """The stream with every pending sum applied (float32)."""
        self._settle()
        return self.residual
