"""The two ends of a decoder as parts: token ids in, logits out.

``lookup``: the residual stream starts as row ``id`` of the embedding table, widened to float32, no multiplier
(python/stride_worker/model.py:250-252). ``linear``: logits are the normed rows times the head matrix, computed in
the compute dtype and returned in float32; a head whose spec names no tensor shares the embedding table
(python/stride_worker/model.py:127-130, 322-341). An architecture that scales its embedding, adds a bias to its
head or caps its logits registers another kind; the model itself does not change.
"""

from __future__ import annotations

from ..csrc import ops
from .base import Embedding, Head, TensorDecl, register_part


class LookupEmbedding(Embedding):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.weight = None

    def declare(self):
        return {self.spec.name: TensorDecl((self.spec.vocab, self.spec.hidden))}

    def bind(self, weights):
        self.weight = weights[self.spec.name]

    def named_tensors(self):
        return {self.spec.name: self.weight}

    def table(self):
        return self.weight

    def forward(self, ctx, out):
        tokens = out.shape[0]
        ops.embed_gather(ctx.token_ids[:tokens], ctx.seq_of_token[:tokens], self.weight, out)


class LinearHead(Head):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.weight = None

    def declare(self):
        return {} if self.spec.name is None else {self.spec.name: TensorDecl((self.spec.vocab, self.spec.hidden))}

    def bind(self, weights, tied=None):
        if self.spec.name is not None:
            self.weight = weights[self.spec.name]
        elif tied is None:
            raise ValueError("the head names no tensor and the embedding offers no table to share")
        else:
            self.weight = tied

    def named_tensors(self):
        return {} if self.spec.name is None else {self.spec.name: self.weight}

    def forward(self, x, out):
        ops.linear(x, self.weight, out)


register_part("embedding", "lookup", LookupEmbedding)
register_part("head", "linear", LinearHead)
