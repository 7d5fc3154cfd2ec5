"""Typed configuration of the Llama 3 dense decoder (``LlamaForCausalLM``).

Keys and defaults follow what the reference reads from config.json
(python/stride_worker/model.py:101-108,173-180 and
crates/stride-model/src/config.rs:213-299): ``num_key_value_heads`` defaults to
the number of query heads, ``head_dim`` to ``hidden_size // num_attention_heads``,
``rms_norm_eps`` to 1e-5, ``rope_theta`` to 10000, ``max_position_embeddings`` to
8192; a missing required key is an error, never a default. Beyond the reference,
``intermediate_size`` and ``tie_word_embeddings`` are read and later checked
against the checkpoint, an activation other than SiLU, MLP biases or an unknown
rope type are refused, and both ``rope_type`` and the older ``type`` key are
understood.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .registry import ConfigError, register_architecture
from .specs import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, RopeScaling,
                    default_schedule)

_REQUIRED = ("hidden_size", "num_attention_heads", "num_hidden_layers", "vocab_size", "intermediate_size")


def _positive_int(d: dict, key: str, default=None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json is missing `{key}`")
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"`{key}` must be a positive integer, got {v!r}")
    return v


def _number(d: dict, key: str, default: float) -> float:
    v = d.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"`{key}` must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_id: tuple = ()
    torch_dtype: Optional[str] = None
    architectures: tuple = ("LlamaForCausalLM",)
    name: str = "unnamed"
    extra: dict = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        for key in _REQUIRED:
            if key not in d:
                raise ConfigError(f"config.json is missing `{key}`")
        hidden = _positive_int(d, "hidden_size")
        nq = _positive_int(d, "num_attention_heads")
        nkv = _positive_int(d, "num_key_value_heads", nq)
        if "head_dim" in d and d["head_dim"] is not None:
            hd = _positive_int(d, "head_dim")
        else:
            if hidden % nq:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {nq} and no head_dim is given")
            hd = hidden // nq
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported by this architecture's feed-forward (silu only)")
        if d.get("mlp_bias", False):
            raise ConfigError("mlp_bias=true is not supported")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)
        known = {f for f in cls.__dataclass_fields__} | {"mlp_bias", "model_type", "_name_or_path"}
        cfg = cls(
            vocab_size=_positive_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(d, "intermediate_size"),
            num_hidden_layers=_positive_int(d, "num_hidden_layers"),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=hd,
            rms_norm_eps=_number(d, "rms_norm_eps", 1e-5),
            rope_theta=_number(d, "rope_theta", 10000.0),
            rope_scaling=_read_rope_scaling(d.get("rope_scaling")),
            max_position_embeddings=_positive_int(d, "max_position_embeddings", 8192),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            hidden_act=act,
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=eos_ids,
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
            architectures=tuple(d.get("architectures") or ("LlamaForCausalLM",)),
            name=str(d.get("_name_or_path", "unnamed")),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @staticmethod
    def complete_from_checkpoint(d: dict, tensor_names: set) -> dict:
        """Two options that the reference settles by what the checkpoint holds, never by config.json
        (python/stride_worker/model.py:127-128,159-169): the head is tied when ``lm_head.weight`` is absent,
        and the q/k/v projections have biases when the bias tensors are there. A config.json that gives the
        key is taken at its word (and checked against the checkpoint at load); one that leaves it out gets it
        from the checkpoint here."""
        if "tie_word_embeddings" not in d:
            d["tie_word_embeddings"] = "lm_head.weight" not in tensor_names
        if "attention_bias" not in d:
            d["attention_bias"] = any(n.endswith(".self_attn.q_proj.bias") for n in tensor_names)
        return d

    def with_max_positions(self, count: int) -> "LlamaConfig":
        """The same model with position tables for ``count`` positions. The rotation is defined for every
        position (its angles do not depend on ``max_position_embeddings``, which only sizes the table), so a
        tool that feeds given tokens may go on past the length the checkpoint names."""
        import dataclasses
        return dataclasses.replace(self, max_position_embeddings=int(count))

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{self.num_attention_heads} query heads do not divide evenly into "
                              f"{self.num_key_value_heads} KV heads")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary embeddings")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")
        for e in self.eos_token_id:
            if not 0 <= e < self.vocab_size:
                raise ConfigError(f"eos_token_id {e} lies outside the vocabulary")

    def to_dict(self) -> dict:
        d = {
            "architectures": list(self.architectures),
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": False,
            "hidden_act": self.hidden_act,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            d["rope_scaling"] = {"rope_type": s.rope_type, "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                                 "high_freq_factor": s.high_freq_factor,
                                 "original_max_position_embeddings": s.original_max_position_embeddings}
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            d["eos_token_id"] = self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d

    # --------------------------------------------------------------- arithmetic
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def params_per_layer(self) -> int:
        """Matrix weights of one layer (crates/stride-model/src/config.rs:122-131)."""
        h = self.hidden_size
        return h * self.q_dim + 2 * h * self.kv_dim + self.q_dim * h + 3 * h * self.intermediate_size

    def total_params(self, with_norms: bool = True) -> int:
        embed = self.vocab_size * self.hidden_size * (1 if self.tie_word_embeddings else 2)
        norms = (2 * self.num_hidden_layers + 1) * self.hidden_size if with_norms else 0
        return self.params_per_layer() * self.num_hidden_layers + embed + norms

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """Keys and values of one token over all layers (config.rs:169-171)."""
        return 2 * self.num_hidden_layers * self.kv_dim * itemsize

    # ------------------------------------------------------------------- layout
    def to_model_spec(self) -> ModelSpec:
        position = PositionSpec(kind="rope", head_dim=self.head_dim, theta=self.rope_theta,
                                max_positions=self.max_position_embeddings, scaling=self.rope_scaling)
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append(LayerSpec(
                kind="pre_norm",
                mixer=MixerSpec(kind="attention", hidden=self.hidden_size, num_heads=self.num_attention_heads,
                                num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                                scale=self.head_dim ** -0.5, window=None, bias=self.attention_bias, position=position,
                                prefix=p + "self_attn."),
                feed_forward=FeedForwardSpec(kind="swiglu", hidden=self.hidden_size, intermediate=self.intermediate_size,
                                             activation=self.hidden_act, prefix=p + "mlp."),
                mixer_norm=NormSpec(kind="rmsnorm", width=self.hidden_size, eps=self.rms_norm_eps,
                                    prefix=p + "input_layernorm."),
                ffn_norm=NormSpec(kind="rmsnorm", width=self.hidden_size, eps=self.rms_norm_eps,
                                  prefix=p + "post_attention_layernorm."),
            ))
        return ModelSpec(
            architecture=self.architectures[0],
            hidden=self.hidden_size,
            vocab=self.vocab_size,
            layers=tuple(layers),
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=NormSpec(kind="rmsnorm", width=self.hidden_size, eps=self.rms_norm_eps, prefix="model.norm."),
            embed_name="model.embed_tokens.weight",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            max_positions=self.max_position_embeddings,
            eos_token_ids=self.eos_token_id,
            bos_token_id=self.bos_token_id,
            ignorable_tensors=("*.rotary_emb.inv_freq",),
            extra=self,
        )


def _read_rope_scaling(raw) -> Optional[RopeScaling]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"rope_scaling must be an object, got {raw!r}")
    kind = raw.get("rope_type", raw.get("type"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise ConfigError(f"rope_scaling type {kind!r} is not supported (llama3 or none)")
    # Defaults of the reference (python/stride_worker/layers.py:57-60).
    s = RopeScaling(
        rope_type="llama3",
        factor=_number(raw, "factor", 8.0),
        low_freq_factor=_number(raw, "low_freq_factor", 1.0),
        high_freq_factor=_number(raw, "high_freq_factor", 4.0),
        original_max_position_embeddings=_positive_int(raw, "original_max_position_embeddings", 8192),
    )
    if s.factor <= 0 or s.high_freq_factor == s.low_freq_factor:
        raise ConfigError("rope_scaling needs factor > 0 and high_freq_factor != low_freq_factor")
    return s


register_architecture("LlamaForCausalLM", LlamaConfig, model_type="llama")
