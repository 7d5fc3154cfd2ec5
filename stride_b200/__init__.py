"""stride_b200: a small, whole LLM inference engine for one NVIDIA B200.

    from stride_b200 import Engine, SamplingParams
    engine = Engine("/path/to/model_dir", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))

Heavy parts (torch, the compiled kernels) load on first use.
"""

__version__ = "0.1.0"

_LAZY = {
    "Engine": ("stride_b200.engine", "Engine"),
    "RequestOutput": ("stride_b200.engine", "RequestOutput"),
    "EngineBusy": ("stride_b200.engine", "EngineBusy"),
    "TraceSession": ("stride_b200.engine", "TraceSession"),
    "write_random_model": ("stride_b200.engine", "write_random_model"),
    "random_model": ("stride_b200.engine", "random_model"),
    "load_model": ("stride_b200.engine", "load_model"),
    "SamplingParams": ("stride_b200.sampling", "SamplingParams"),
    "EngineConfig": ("stride_b200.config", "EngineConfig"),
    "LlamaConfig": ("stride_b200.config", "LlamaConfig"),
    "load_config": ("stride_b200.config", "load_config"),
    "config_from_dict": ("stride_b200.config", "config_from_dict"),
    "register_architecture": ("stride_b200.config", "register_architecture"),
    "register_part": ("stride_b200.parts", "register_part"),
    "preset": ("stride_b200.config", "preset"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(f"module 'stride_b200' has no attribute {name!r}")


__all__ = sorted(_LAZY)
