"""What a model is made of, as data.

A model is a list of layers and a list that says in which order they run. A
layer is an arrangement of four parts: a mixer (attention here), a feed-forward,
and the norms before them. Each part is described by a small frozen record that
carries every size and constant the part needs; the record's ``kind`` selects
the implementation from the part registry (``stride_b200.parts``). No part knows
which architecture it serves, and layers of one model may use different kinds.

The records also carry the checkpoint prefix under which a part finds its
tensors, so that tensor naming stays with the architecture that defines it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of rotary embeddings (``rope_scaling`` in config.json)."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer. kind ``rope`` | ``none``."""
    kind: str
    head_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: Optional[RopeScaling] = None
    params: tuple = ()          # free-form (key, value) pairs for other kinds


@dataclass(frozen=True)
class NormSpec:
    """kind ``rmsnorm``: y = x * rsqrt(mean(x^2) + eps) * weight."""
    kind: str
    width: int
    eps: float
    prefix: str                 # e.g. "model.layers.0.input_layernorm."
    params: tuple = ()


@dataclass(frozen=True)
class MixerSpec:
    """kind ``attention``: grouped-query attention over the paged cache.

    ``window`` of None keeps every key; an integer W lets a token read only its
    last W keys (its own included).
    """
    kind: str
    hidden: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    bias: bool = False
    position: Optional[PositionSpec] = None
    prefix: str = ""            # e.g. "model.layers.0.self_attn."
    params: tuple = ()


@dataclass(frozen=True)
class FeedForwardSpec:
    """kind ``swiglu``: down(act(gate(x)) * up(x))."""
    kind: str
    hidden: int
    intermediate: int = 0
    activation: str = "silu"
    prefix: str = ""            # e.g. "model.layers.0.mlp."
    params: tuple = ()


@dataclass(frozen=True)
class LayerSpec:
    """kind ``pre_norm``: x += mixer(norm(x)); x += ffn(norm(x))."""
    kind: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    ffn_norm: NormSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache`` names the cache slot (and state slot) that the
    run's mixer uses; two runs with the same slot share keys and values, and
    ``writes_cache=False`` makes a run read what another run wrote."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the first residual stream. kind ``lookup``: row ``id`` of the table ``name``
    [vocab, hidden], no scaling (python/stride_worker/model.py:250-252)."""
    kind: str
    vocab: int
    hidden: int
    name: str                   # checkpoint name of the table
    params: tuple = ()          # free-form (key, value) pairs for other kinds (a multiplier, say)


@dataclass(frozen=True)
class HeadSpec:
    """How the normed last hidden states become logits. kind ``linear``: ``x @ W.T`` in the compute dtype with a
    float32 result; ``name`` None ties W to the embedding table (python/stride_worker/model.py:127-130,322-341)."""
    kind: str
    vocab: int
    hidden: int
    name: Optional[str]
    params: tuple = ()          # free-form (key, value) pairs for other kinds (a bias, a cap on the logits)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    layers: tuple               # of LayerSpec
    schedule: tuple             # of ScheduleEntry
    final_norm: NormSpec
    embed_name: str             # checkpoint name of the embedding table
    head_name: Optional[str]    # checkpoint name of the output head; None: tied to the embedding
    max_positions: int
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    ignorable_tensors: tuple = ()   # glob patterns of checkpoint tensors that may be present and are not read
    extra: Any = field(default=None, compare=False)
    # The two ends of the model are parts like the rest. Left out, they are the plain kinds built from the two
    # names above: a table lookup and a linear head.
    embedding: Optional[EmbeddingSpec] = None
    head: Optional[HeadSpec] = None

    def embedding_spec(self) -> EmbeddingSpec:
        return self.embedding or EmbeddingSpec("lookup", self.vocab, self.hidden, self.embed_name)

    def head_spec(self) -> HeadSpec:
        return self.head or HeadSpec("linear", self.vocab, self.hidden, self.head_name)

    @property
    def num_cache_slots(self) -> int:
        return 1 + max(e.cache for e in self.schedule) if self.schedule else 0


def default_schedule(num_layers: int) -> tuple:
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(num_layers))
