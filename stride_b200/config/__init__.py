from .engine import DTYPES, EngineConfig
from .llama import LlamaConfig
from .memory import B200_MEMORY_BYTES, MemoryPlan, PlanError, plan_memory
from .presets import PRESETS, preset
from .registry import (ConfigError, config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .specs import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, RopeScaling, ScheduleEntry,
                    default_schedule)

__all__ = [
    "DTYPES", "EngineConfig", "LlamaConfig", "MemoryPlan", "PlanError", "plan_memory", "B200_MEMORY_BYTES", "PRESETS", "preset", "ConfigError", "config_class_for", "config_from_dict",
    "load_config", "register_architecture", "registered_architectures", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec", "LayerSpec", "MixerSpec",
    "ModelSpec", "NormSpec", "PositionSpec", "RopeScaling", "ScheduleEntry", "default_schedule",
]
