"""Shared test material: tiny configurations, seeded weights and comparisons.

Nothing here imports the product package, so the plain implementation and the
golden script can use it without touching the code under test.
"""

from __future__ import annotations

import json
import os

import torch

# Three tiny Llama 3 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 192,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "intermediate_size": 256,
    "vocab_size": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}

# Odd sizes: a prime vocabulary, a width that is no power of two, head_dim 48,
# as many key heads as query heads, head_dim * heads != hidden.
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 1,
    "hidden_size": 88,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "intermediate_size": 136,
    "vocab_size": 251,
    "rope_theta": 25000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 4.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 2.0,
        "original_max_position_embeddings": 32,
    },
    "rms_norm_eps": 3e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
    "hidden_act": "silu",
}

# Head size 128 and a group of 4, the sizes that the tensor-core attention kernels and the
# tcgen05 matrix product take, so that whole-model runs go through them too.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 192,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "head_dim": 128,
    "intermediate_size": 320,
    "vocab_size": 515,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 128,
    },
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
    "hidden_act": "silu",
}

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 16}


def geometry(cfg: dict):
    nq = int(cfg["num_attention_heads"])
    nkv = int(cfg.get("num_key_value_heads", nq))
    hd = int(cfg.get("head_dim", int(cfg["hidden_size"]) // nq))
    return nq, nkv, hd


def seeded_state(cfg: dict, seed: int, std: float = 0.02, norm_jitter: float = 0.1) -> dict:
    """float32 weights N(0, std) in checkpoint-name order from one generator;
    norm weights are 1 + N(0, norm_jitter) so that a dropped norm weight shows."""
    g = torch.Generator().manual_seed(seed)
    nq, nkv, hd = geometry(cfg)
    H, I, V = int(cfg["hidden_size"]), int(cfg["intermediate_size"]), int(cfg["vocab_size"])

    def mat(rows, cols):
        return torch.randn(rows, cols, generator=g, dtype=torch.float32) * std

    def norm():
        return 1.0 + torch.randn(H, generator=g, dtype=torch.float32) * norm_jitter

    state = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(int(cfg["num_hidden_layers"])):
        p = f"model.layers.{i}"
        state[f"{p}.input_layernorm.weight"] = norm()
        state[f"{p}.self_attn.q_proj.weight"] = mat(nq * hd, H)
        state[f"{p}.self_attn.k_proj.weight"] = mat(nkv * hd, H)
        state[f"{p}.self_attn.v_proj.weight"] = mat(nkv * hd, H)
        state[f"{p}.self_attn.o_proj.weight"] = mat(H, nq * hd)
        state[f"{p}.post_attention_layernorm.weight"] = norm()
        state[f"{p}.mlp.gate_proj.weight"] = mat(I, H)
        state[f"{p}.mlp.up_proj.weight"] = mat(I, H)
        state[f"{p}.mlp.down_proj.weight"] = mat(H, I)
    state["model.norm.weight"] = norm()
    if not cfg.get("tie_word_embeddings", False):
        state["lm_head.weight"] = mat(V, H)
    return state


def seeded_biases(cfg: dict, seed: int, std: float = 0.1) -> dict:
    """q/k/v projection biases N(0, std) for every layer (the reference uses them when the checkpoint has them,
    python/stride_worker/model.py:159-169)."""
    g = torch.Generator().manual_seed(seed)
    nq, nkv, hd = geometry(cfg)
    out = {}
    for i in range(int(cfg["num_hidden_layers"])):
        for proj, rows in (("q", nq * hd), ("k", nkv * hd), ("v", nkv * hd)):
            out[f"model.layers.{i}.self_attn.{proj}_proj.bias"] = torch.randn(rows, generator=g, dtype=torch.float32) * std
    return out


def seeded_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def write_model_dir(path: str, cfg: dict, state: dict, dtype=torch.float32) -> str:
    """A model folder for the engine, written with the ``safetensors`` package
    (not with the product's own writer)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in state.items()},
              os.path.join(path, "model.safetensors"))
    return path


def read_model_dir(path: str):
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(path, "model.safetensors"))


# Thresholds in the manner of python/stride_worker/diagnose/equivalence.py:40-54
# (cosine floors per dtype) plus an absolute bound scaled to the logits' size.
COSINE_FLOOR = {"float32": 0.9999999, "bfloat16": 0.9995}
REL_MAX_ABS = {"float32": 2e-5, "bfloat16": 4e-2}


def compare_logits(got: torch.Tensor, want: torch.Tensor, dtype: str):
    """Returns (ok, message). Rows are compared in float64: the worst cosine
    must stay above the dtype's floor and the largest absolute difference below
    the dtype's bound relative to the largest reference logit."""
    a = got.to(torch.float64).reshape(-1, got.shape[-1])
    b = want.to(torch.float64).reshape(-1, want.shape[-1])
    if a.shape != b.shape:
        return False, f"shape {tuple(a.shape)} != {tuple(b.shape)}"
    if not torch.isfinite(a).all():
        return False, "non-finite logits"
    cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
    diff = (a - b).abs()
    scale = b.abs().max().clamp_min(1e-12)
    worst = int(diff.max(dim=-1).values.argmax())
    msg = (f"min cosine {cos.min():.9f} (row {int(cos.argmin())}), max abs diff {diff.max():.3e} "
           f"(row {worst}), reference scale {scale:.3e}")
    ok = bool(cos.min() >= COSINE_FLOOR[dtype]) and bool(diff.max() <= REL_MAX_ABS[dtype] * scale)
    return ok, msg
