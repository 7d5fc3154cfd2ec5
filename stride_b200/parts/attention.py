"""Grouped-query attention over the paged cache.

q/k/v projections (fused into one matrix product at load time), position
encoding and cache write, attention of every token over its request's pages,
output projection: python/stride_worker/model.py:258-299 with the attention rule
of python/stride_worker/layers.py:109-149. Biases are used when the spec says so.
A window (not used by Llama 3) limits each token to its last W keys.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheRequest, Mixer, Projection, TensorDecl, build_part, register_part


class PagedAttention(Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads do not group into {s.num_kv_heads} KV heads")
        if s.head_dim % 16 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim} is not supported by the attention kernels "
                             "(multiples of 16 up to 256 are)")
        if s.window is not None and s.window <= 0:
            raise ValueError("an attention window must be positive")
        self.hidden = s.hidden
        self.nq, self.nkv, self.hd = s.num_heads, s.num_kv_heads, s.head_dim
        self.q_dim, self.kv_dim = self.nq * self.hd, self.nkv * self.hd
        self.qkv_dim = self.q_dim + 2 * self.kv_dim
        self.scale = float(s.scale)
        self.window = 0 if s.window is None else int(s.window)
        self.position = build_part("position", s.position, runtime)
        self.w_qkv = self.w_o = self.bias = None
        self._fast = ops.fast_attention_supported(runtime.dtype, self.nq, self.nkv, self.hd)

    # ----------------------------------------------------------------- weights
    def _names(self):
        p = self.spec.prefix
        return {k: f"{p}{k}_proj.weight" for k in "qkvo"}, {k: f"{p}{k}_proj.bias" for k in "qkv"}

    def declare(self):
        w, b = self._names()
        d = {w["q"]: TensorDecl((self.q_dim, self.hidden)), w["k"]: TensorDecl((self.kv_dim, self.hidden)),
             w["v"]: TensorDecl((self.kv_dim, self.hidden)), w["o"]: TensorDecl((self.hidden, self.q_dim))}
        if self.spec.bias:
            d[b["q"]] = TensorDecl((self.q_dim,), "vector")
            d[b["k"]] = TensorDecl((self.kv_dim,), "vector")
            d[b["v"]] = TensorDecl((self.kv_dim,), "vector")
        d.update(self.position.declare())          # a position encoding may have tensors of its own
        return d

    def bind(self, weights):
        w, b = self._names()
        self.w_qkv = torch.cat([weights[w["q"]], weights[w["k"]], weights[w["v"]]], dim=0).contiguous()
        self.w_o = weights[w["o"]]
        if self.spec.bias:
            self.bias = torch.cat([weights[b["q"]], weights[b["k"]], weights[b["v"]]]).contiguous()
        self.position.bind(weights)

    def named_tensors(self):
        w, b = self._names()
        q, k = self.q_dim, self.q_dim + self.kv_dim
        out = {w["q"]: self.w_qkv[:q], w["k"]: self.w_qkv[q:k], w["v"]: self.w_qkv[k:], w["o"]: self.w_o}
        if self.bias is not None:
            out.update({b["q"]: self.bias[:q], b["k"]: self.bias[q:k], b["v"]: self.bias[k:]})
        out.update(self.position.named_tensors())
        return out

    # ------------------------------------------------------------------- cache
    def cache_request(self):
        return CacheRequest(self.nkv, self.hd, self.spec.window)

    # ----------------------------------------------------------------- forward
    lazy_output = True
    accepts_folded = True

    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens = x.shape[0]
        qkv = self.rt.buffer("qkv", tokens, self.qkv_dim)
        folded = x if isinstance(x, ops.FoldedNorm) else None
        if not self._project_and_rotate(folded.xt if folded else x, qkv, ctx, cache, tokens, folded):
            if folded:
                x = folded.tensor()
            ops.linear(x, self.w_qkv, qkv)
            self.position.encode_and_store(qkv, self.bias, ctx, cache, self.nq, self.nkv, self.hd)
        attn = self.rt.buffer("attn", tokens, self.q_dim)
        self._attend(qkv, attn, ctx, cache, tokens)
        if lazy_output:
            return Projection(attn, self.w_o)          # the residual stream runs it, with the sum and norm that follow if it can
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(attn, self.w_o, out)
        return out


    def _project_and_rotate(self, x, qkv, ctx, cache, tokens, folded=None) -> bool:
        """A decode step's projection with the position encoding and the cache write in its epilogue, when the
        position part says that what it does is the standard rotation. False: nothing was done."""
        if tokens > max(ops.TC_GEMM_MAX_TOKENS, ops.ROWS_GEMM_MAX_TOKENS) or x.dtype != torch.bfloat16:
            return False
        tables = self.position.rotation_tables()
        if tables is None:
            return False
        cos, sin, rotate = tables
        slots = ctx.slot_mapping[cache.group][:tokens] if cache.writes else None
        if tokens > ops.TC_GEMM_MAX_TOKENS:         # the tokens-as-rows kernel, where the policy sends steps of this size to it
            return ops.rows_wanted(tokens) and ops.linear_rows_qkv_rope(
                x, self.w_qkv, qkv, self.bias, ctx.positions[:tokens], slots, cos, sin, cache.k_pages, cache.v_pages, self.nq, self.nkv,
                self.hd, cache.page_size, rotate, folded)
        return ops.linear_qkv_rope(x, self.w_qkv, qkv, self.bias, ctx.positions[:tokens], slots, cos, sin, cache.k_pages,
                                   cache.v_pages, self.nq, self.nkv, self.hd, cache.page_size, rotate, folded)

    def _attend(self, qkv, attn, ctx, cache, tokens):
        table = ctx.block_table[cache.group]
        geometry = (self.nq, self.nkv, self.hd, cache.page_size, self.scale, self.window)
        if not self._fast:
            # the exact kernel: the whole 32-bit path, and bfloat16 sizes the tensor-core kernels refuse
            ops.paged_attention(qkv, self.qkv_dim, attn, cache.k_pages, cache.v_pages, table, ctx.seq_of_token[:tokens],
                                ctx.positions[:tokens], *geometry)
            return
        split = min(ctx.decode_tail_start, tokens)          # portions before, single decoded tokens after
        if split > 0:
            args = (qkv[:split], self.qkv_dim, attn[:split], cache.k_pages, cache.v_pages, table, ctx.q_start, ctx.q_len,
                    ctx.ctx_len, ctx.decode_tail_seq, *geometry)
            # tcgen05 kernel first; the mma.sync kernel takes what it refuses (odd page sizes)
            if not (ops.TC_ATTENTION and ops.paged_attention_prefill_tc(*args)):
                ops.paged_attention_prefill(*args)
        if tokens > split:
            n = tokens - split
            scratch = self.rt.scratch("attention_splits", ops.decode_scratch_floats(n, self.nq, self.nkv, self.hd, ctx.context_bound))
            ops.paged_attention_decode(qkv[split:tokens], self.qkv_dim, attn[split:tokens], cache.k_pages, cache.v_pages, table,
                                       ctx.seq_of_token[split:tokens], ctx.positions[split:tokens], scratch, *geometry,
                                       ctx.context_bound)


register_part("mixer", "attention", PagedAttention)
