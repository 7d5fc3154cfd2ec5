"""A plain, slow Llama 3 decoder: whole sequences, no cache, one function per part.

This file is the yardstick of the test-suite. It is written from the formulas
of the reference project (each function cites the file and lines it restates)
and shares no code with the ``stride_b200`` package: it never imports it.
Everything runs where the weights live (the CPU in most tests; a CUDA device
for the models that are too wide for it) in the dtype that the caller names
(float32 by default, float64 for a reference that rounding cannot blur). The
rotation tables are always computed on the CPU in float32 and then moved.

Weights are a plain ``dict`` from checkpoint tensor names to tensors, with the
names of ``python/stride_worker/model.py:120-171``.
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w``; the weight multiplies after the
    normalisation (python/stride_worker/layers.py:24-35)."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight.to(x.dtype)


# --------------------------------------------------------------------------- rope
def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """Inverse frequencies in float32, with the llama3 three-band rescaling
    when ``scaling['rope_type'] == 'llama3'`` (python/stride_worker/layers.py:52-77)."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    kind = None
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
    if kind == "llama3":
        factor = float(scaling.get("factor", 8.0))
        low = float(scaling.get("low_freq_factor", 1.0))
        high = float(scaling.get("high_freq_factor", 4.0))
        original = int(scaling.get("original_max_position_embeddings", 8192))
        wavelength = 2 * math.pi / inv_freq
        low_wavelength = original / low
        high_wavelength = original / high
        scaled = inv_freq / factor
        smooth = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
        interpolated = (1 - smooth) * scaled + smooth * inv_freq
        inv_freq = torch.where(wavelength > low_wavelength, scaled, inv_freq)
        middle = (wavelength <= low_wavelength) & (wavelength >= high_wavelength)
        inv_freq = torch.where(middle, interpolated, inv_freq)
    return inv_freq


def rope_tables(head_dim: int, positions: torch.Tensor, theta: float,
                scaling: dict | None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of ``position * inv_freq``, the half-width table repeated
    twice along the last axis (python/stride_worker/layers.py:79-82). Angles
    are float32 products, as in the reference's table."""
    inv_freq = rope_inv_freq(head_dim, theta, scaling)
    freqs = torch.outer(positions.to(torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(-second half, first half) (python/stride_worker/layers.py:85-87)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` for x of shape [n, heads, head_dim]
    (python/stride_worker/layers.py:104-106)."""
    c = cos.unsqueeze(1).to(x.dtype)
    s = sin.unsqueeze(1).to(x.dtype)
    return x * c + rotate_half(x) * s


# ---------------------------------------------------------------------- attention
def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None) -> torch.Tensor:
    """softmax(q k^T * scale + mask) v for one whole sequence.

    q is [n, nq, hd], k and v are [n, nkv, hd]; query head h reads key head
    ``h // (nq // nkv)`` and query i sees keys ``j <= i``
    (python/stride_worker/layers.py:128-149). ``window`` (not used by Llama 3)
    further limits a query to its last ``window`` keys, ``j > i - window``.
    """
    n, nq, hd = q.shape
    nkv = k.shape[1]
    if nq % nkv:
        raise ValueError(f"{nq} query heads do not group into {nkv} KV heads")
    group = nq // nkv
    out = torch.empty_like(q)
    i = torch.arange(n, device=q.device).unsqueeze(1)
    j = torch.arange(n, device=q.device).unsqueeze(0)
    allowed = j <= i
    if window is not None:
        allowed &= j > i - window
    for h in range(nq):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        scores = (q[:, h, :] @ kh.T) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ vh
    return out


# --------------------------------------------------------------------------- ffn
def swiglu(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))`` with ``silu(z) = z * sigmoid(z)``
    (python/stride_worker/layers.py:152-161)."""
    g = x @ gate.T
    u = x @ up.T
    return ((g * torch.sigmoid(g)) * u) @ down.T


# ------------------------------------------------------------------------- blocks
def attention_block(x, w, prefix, cfg, cos, sin, window=None):
    """q/k/v projections (bias only if the checkpoint has one), rotation of q and
    k, attention, output projection (python/stride_worker/model.py:258-299)."""
    nq = int(cfg["num_attention_heads"])
    nkv = int(cfg.get("num_key_value_heads", nq))
    hd = int(cfg.get("head_dim", int(cfg["hidden_size"]) // nq))

    def proj(name):
        y = x @ w[f"{prefix}.self_attn.{name}.weight"].T
        bias = w.get(f"{prefix}.self_attn.{name}.bias")
        return y if bias is None else y + bias

    q = proj("q_proj").view(-1, nq, hd)
    k = proj("k_proj").view(-1, nkv, hd)
    v = proj("v_proj").view(-1, nkv, hd)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    a = causal_attention(q, k, v, hd ** -0.5, window)
    return a.reshape(-1, nq * hd) @ w[f"{prefix}.self_attn.o_proj.weight"].T


def decoder_layer(x, w, i, cfg, cos, sin):
    """Pre-norm block with two residual sums (python/stride_worker/model.py:254-310)."""
    p = f"model.layers.{i}"
    eps = float(cfg.get("rms_norm_eps", 1e-5))
    h = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p, cfg, cos, sin)
    h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
    x = x + swiglu(h, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                   w[f"{p}.mlp.down_proj.weight"])
    return x


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float32, hidden_states: list | None = None):
    """Logits [n, vocab] at every position of one whole sequence.

    Embedding gather, the layers, the final norm and the output head, which is
    the embedding table when the checkpoint has no ``lm_head.weight``
    (python/stride_worker/model.py:120-130, 250-341).
    """
    w = {k: t.to(dtype) for k, t in weights.items()}
    device = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(tokens, dtype=torch.long).to(device)
    nq = int(cfg["num_attention_heads"])
    hd = int(cfg.get("head_dim", int(cfg["hidden_size"]) // nq))
    cos, sin = rope_tables(hd, torch.arange(len(ids)), float(cfg.get("rope_theta", 10000.0)),
                           cfg.get("rope_scaling"))
    cos, sin = cos.to(device), sin.to(device)
    x = w["model.embed_tokens.weight"][ids]
    for i in range(int(cfg["num_hidden_layers"])):
        x = decoder_layer(x, w, i, cfg, cos, sin)
        if hidden_states is not None:
            hidden_states.append(x.clone())
    x = rms_norm(x, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-5)))
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return x @ head.T


def greedy_generate(cfg: dict, weights: dict, prompt, n_new: int, dtype=torch.float32) -> list[int]:
    """Append ``n_new`` argmax tokens, recomputing the whole sequence each time."""
    tokens = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, weights, tokens, dtype)
        tokens.append(argmax(logits[-1]))
    return tokens[len(prompt):]


# ----------------------------------------------------------------------- sampling
MASK64 = (1 << 64) - 1


class XorShiftRng:
    """xorshift64* seeded through splitmix64 (crates/stride-backend/src/sampler.rs:18-46)."""

    def __init__(self, seed: int):
        z = (seed + 0x9E3779B97F4A7C15) & MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        self.state = max(z ^ (z >> 31), 1)

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x = (x ^ (x << 25)) & MASK64
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & MASK64

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


def argmax(logits) -> int:
    """Index of the first maximum (crates/stride-backend/src/sampler.rs:157-165)."""
    best = 0
    values = [float(v) for v in logits]
    for i, v in enumerate(values):
        if v > values[best]:
            best = i
    return best


def softmax(logits: torch.Tensor) -> torch.Tensor:
    """Max-subtracted softmax in float32; all ``-inf`` gives the uniform
    distribution (crates/stride-backend/src/sampler.rs:169-183)."""
    logits = logits.to(torch.float32)
    m = logits.max()
    if not torch.isfinite(m):
        return torch.full_like(logits, 1.0 / logits.numel())
    e = torch.exp(logits - m)
    s = e.sum()
    return e / s if s > 0 else e


def sample(logits: torch.Tensor, rng: XorShiftRng, temperature: float = 1.0, top_k: int | None = None,
           top_p: float = 1.0, eos: int | None = None, min_tokens: int = 0, generated: int = 0) -> int:
    """One draw as the reference makes it: EOS suppression below ``min_tokens``,
    greedy when temperature is 0 or top_k is 1, else temperature, a single
    descending ranking, top-k then nucleus cut, and a walk down the kept ranking
    with ``u * kept_mass`` (crates/stride-backend/src/sampler.rs:74-146)."""
    work = logits.to(torch.float32).clone()
    if eos is not None and generated < min_tokens and 0 <= eos < work.numel():
        work[eos] = float("-inf")
    if temperature == 0.0 or top_k == 1:
        return argmax(work)
    if temperature > 0.0 and abs(temperature - 1.0) > 1.1920929e-07:
        work = work / temperature
    probs = softmax(work)
    order = sorted(range(probs.numel()), key=lambda i: -float(probs[i]))
    keep = len(order)
    if top_k is not None:
        keep = min(keep, top_k)
    if top_p < 1.0:
        cumulative, nucleus = 0.0, 0
        for rank, idx in enumerate(order):
            cumulative += float(probs[idx])
            nucleus = rank + 1
            if cumulative >= top_p:
                break
        keep = min(keep, max(nucleus, 1))
    total = sum(float(probs[i]) for i in order[:keep])
    if total <= 0.0 or not math.isfinite(total):
        return order[0]
    target = rng.next_f32() * total
    for idx in order[:keep]:
        target -= float(probs[idx])
        if target <= 0.0:
            return idx
    return order[keep - 1]


# ------------------------------------------------------------------- prefix hashing
FNV_OFFSET = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3


def _fnv1a(acc: int, data: bytes) -> int:
    for b in data:
        acc = ((acc ^ b) * FNV_PRIME) & MASK64
    return acc


def prefix_chain(tenant: str, tokens, page_size: int) -> list[int]:
    """FNV-1a chain over full pages: the root hashes the tenant's bytes, each
    page hashes its parent (8 little-endian bytes, restarting from the offset)
    then its tokens (4 little-endian bytes each)
    (crates/stride-kvcache/src/hash.rs:15-58)."""
    parent = _fnv1a(FNV_OFFSET, tenant.encode("utf-8"))
    out = []
    for start in range(0, len(tokens) - page_size + 1, page_size):
        acc = _fnv1a(FNV_OFFSET, parent.to_bytes(8, "little"))
        for t in tokens[start:start + page_size]:
            acc = _fnv1a(acc, int(t).to_bytes(4, "little"))
        parent = acc
        out.append(acc)
    return out
