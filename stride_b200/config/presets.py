"""Named Llama 3 shapes, as config.json dictionaries: the tiny shapes used
for correctness runs (tiny-d has the head size and widths that the tensor-core
kernels take) and the 8B / 3B / 70B shapes used for measurements. The
reference keeps such presets in crates/stride-model/src/presets.rs:73-91."""

from __future__ import annotations

import copy


def _llama3_scaling(factor: float, original: int) -> dict:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": original}


def _llama(layers, hidden, heads, kv_heads, head_dim, inter, vocab, theta, scaling, eps, tied, max_pos) -> dict:
    d = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "hidden_size": hidden,
         "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter,
         "vocab_size": vocab, "rope_theta": theta, "rms_norm_eps": eps, "tie_word_embeddings": tied,
         "max_position_embeddings": max_pos, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False}
    if scaling:
        d["rope_scaling"] = scaling
    return d


PRESETS = {
    "tiny-a": _llama(2, 64, 4, 2, 16, 192, 256, 10000.0, None, 1e-5, False, 256),
    "tiny-b": _llama(3, 96, 3, 1, 32, 256, 384, 500000.0, _llama3_scaling(8.0, 64), 1e-6, True, 512),
    "tiny-d": _llama(2, 192, 4, 2, 128, 384, 515, 500000.0, _llama3_scaling(8.0, 128), 1e-5, False, 2048),
    "llama3.1-8b": _llama(32, 4096, 32, 8, 128, 14336, 128256, 500000.0, _llama3_scaling(8.0, 8192), 1e-5, False, 131072),
    "llama3.2-3b": _llama(28, 3072, 24, 8, 128, 8192, 128256, 500000.0, _llama3_scaling(32.0, 8192), 1e-5, True, 131072),
    "llama3.1-70b": _llama(80, 8192, 64, 8, 128, 28672, 128256, 500000.0, _llama3_scaling(8.0, 8192), 1e-5, False, 131072),
}


def preset(name: str) -> dict:
    try:
        return copy.deepcopy(PRESETS[name])
    except KeyError:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}") from None
