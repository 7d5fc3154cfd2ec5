"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``
(python/stride_worker/layers.py:152-161). Gate and up are one matrix product
(their weights are stacked at load time); SiLU and the product run in float32.

In bfloat16, when the inner width allows it, the stacked weight alternates 64 rows
of gate and 64 rows of up, so that a 128-row tile of the decode product holds both
halves of 64 activations and its epilogue can apply SiLU and the product itself;
``silu_mul`` reads the same layout after the library product of a prefill."""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, Projection, TensorDecl, register_part


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """[2 * inter, hidden]: ``block`` rows of gate, ``block`` rows of up, and so on (block == inter: plain stacking)."""
    inter, hidden = gate.shape
    return torch.stack([gate.view(inter // block, block, hidden), up.view(inter // block, block, hidden)], dim=1) \
        .reshape(2 * inter, hidden).contiguous()


class SwiGLU(FeedForward):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported by the swiglu kernel (silu only)")
        self.hidden, self.inter = spec.hidden, spec.intermediate
        self.w_gate_up = self.w_down = None

    def _names(self):
        p = self.spec.prefix
        return p + "gate_proj.weight", p + "up_proj.weight", p + "down_proj.weight"

    def declare(self):
        g, u, d = self._names()
        return {g: TensorDecl((self.inter, self.hidden)), u: TensorDecl((self.inter, self.hidden)),
                d: TensorDecl((self.hidden, self.inter))}

    def bind(self, weights):
        g, u, d = self._names()
        gate, up = weights[g], weights[u]
        self.block = ops.GATED_BLOCK if (gate.dtype == torch.bfloat16 and self.inter % ops.GATED_BLOCK == 0) else self.inter
        self.w_gate_up = interleave_gate_up(gate, up, self.block)
        self.w_down = weights[d]

    def named_tensors(self):
        g, u, d = self._names()
        blocks = self.w_gate_up.view(self.inter // self.block, 2, self.block, self.hidden)
        return {g: blocks[:, 0].reshape(self.inter, self.hidden), u: blocks[:, 1].reshape(self.inter, self.hidden), d: self.w_down}

    lazy_output = True
    accepts_folded = True

    def forward(self, x, ctx, lazy_output: bool = False):
        tokens = x.shape[0]
        act = self.rt.buffer("ffn_act", tokens, self.inter)
        folded = x if isinstance(x, ops.FoldedNorm) else None
        gated = self.block == ops.GATED_BLOCK and (
            ops.linear_gated_tc(folded.xt if folded else x, self.w_gate_up, act, folded)
            or (ops.rows_wanted(tokens) and ops.linear_rows_gated(folded.xt if folded else x, self.w_gate_up, act, folded)))
        if not gated:
            if folded:
                x = folded.tensor()
            gate_up = self.rt.buffer("gate_up", tokens, 2 * self.inter)
            ops.linear(x, self.w_gate_up, gate_up)
            ops.silu_mul(gate_up, act, self.block)
        if lazy_output:
            return Projection(act, self.w_down)        # the residual stream runs it, with the sum and norm that follow if it can
        out = self.rt.buffer("ffn_out", tokens, self.hidden)
        ops.linear(act, self.w_down, out)
        return out


register_part("feed_forward", "swiglu", SwiGLU)
