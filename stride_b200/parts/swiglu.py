"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``
(python/stride_worker/layers.py:152-161). Gate and up are one matrix product
(their weights are stacked at load time); SiLU and the product run in float32."""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, TensorDecl, register_part


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
        self.w_gate_up = torch.cat([weights[g], weights[u]], dim=0).contiguous()
        self.w_down = weights[d]

    def named_tensors(self):
        g, u, d = self._names()
        return {g: self.w_gate_up[:self.inter], u: self.w_gate_up[self.inter:], d: self.w_down}

    def forward(self, x, ctx):
        tokens = x.shape[0]
        gate_up = self.rt.buffer("gate_up", tokens, 2 * self.inter)
        ops.linear(x, self.w_gate_up, gate_up)
        act = self.rt.buffer("ffn_act", tokens, self.inter)
        ops.silu_mul(gate_up, act)
        out = self.rt.buffer("ffn_out", tokens, self.hidden)
        ops.linear(act, self.w_down, out)
        return out


register_part("feed_forward", "swiglu", SwiGLU)
