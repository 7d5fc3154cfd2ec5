"""From a model folder (or a configuration and a seed) to a model on the device
with its cache attached."""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch

from ..cache import CacheManager, DeviceCache
from ..config import DTYPES, config_from_dict, load_config
from ..csrc import ops
from ..parts import DecoderModel, Runtime
from ..weights import RandomSource, SafetensorsSource, save_file


def build_model(config, source, dtype: str, device="cuda", token_capacity: int = 2048, row_capacity: int = 256):
    """``config``: a typed configuration (anything with ``to_model_spec``)."""
    ops.require_device()
    runtime = Runtime(device, DTYPES[dtype], token_capacity, row_capacity)
    model = DecoderModel(config.to_model_spec(), runtime)
    if source is None:
        raise ValueError("a weight source is needed")
    model.load(source)
    return model


def load_model(model_dir: str, dtype: str = "bfloat16", device="cuda", token_capacity: int = 2048, row_capacity: int = 256,
               min_positions: int = 0):
    """``min_positions``: position tables for at least this many positions, where the configuration can give them
    (``with_max_positions``), even if the checkpoint names a shorter length."""
    source = SafetensorsSource(model_dir)
    config = load_config(model_dir, tensor_names=source.names())
    spec_positions = getattr(config, "max_position_embeddings", None)
    if min_positions and spec_positions is not None and spec_positions < min_positions and hasattr(config, "with_max_positions"):
        config = config.with_max_positions(min_positions)
    return config, build_model(config, source, dtype, device, token_capacity, row_capacity)


def random_model(config, seed: int, dtype: str = "bfloat16", device="cuda", token_capacity: int = 2048,
                 row_capacity: int = 256, std: float = 0.02, vector_jitter: float = 0.0):
    """Random weights drawn on the device, through the same declarations and
    checks as a checkpoint."""
    ops.require_device()
    runtime = Runtime(device, DTYPES[dtype], token_capacity, row_capacity)
    model = DecoderModel(config.to_model_spec(), runtime)
    source = RandomSource(model.declare(), seed, std=std, vector_jitter=vector_jitter, stored_dtype=DTYPES[dtype],
                          device=str(runtime.device))
    model.load(source)
    return model


def write_random_model(config, seed: int, out_dir: str, stored_dtype: str = "bfloat16", std: float = 0.02,
                       vector_jitter: float = 0.0) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` with seeded
    random weights (drawn on the CPU; needs no GPU)."""
    os.makedirs(out_dir, exist_ok=True)
    declared = _declarations(config)
    source = RandomSource(declared, seed, std=std, vector_jitter=vector_jitter, stored_dtype=DTYPES[stored_dtype],
                          device="cpu")
    tensors = {name: source.read(name) for name in declared if not declared[name].optional}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "generator": "stride_b200.write_random_model", "seed": seed})
    return out_dir


def _declarations(config) -> dict:
    """The tensors a model of this configuration reads, without touching a device."""
    runtime = Runtime("meta", torch.float32, 1, 1)
    return DecoderModel(config.to_model_spec(), runtime).declare()


def footprint(config, dtype: str = "bfloat16") -> dict:
    """What a model of this configuration needs in bytes, read from its own parts without touching a device: the
    declared tensors (matrices in the compute dtype, vectors and tables in 32 bits, as the loader keeps them),
    what its mixers keep per token in pages, and the state of fixed size per request. Works for any registered
    architecture, since it asks the parts and not the configuration class."""
    import math

    from ..cache import plan_groups
    item = torch.empty((), dtype=DTYPES[dtype]).element_size()
    model = DecoderModel(config.to_model_spec(), Runtime("meta", DTYPES[dtype], 1, 1))
    weights = sum(math.prod(d.shape) * (item if d.role == "matrix" else 4) for d in model.declare().values() if not d.optional)
    requests = model.cache_requests()
    per_token = sum(g.elements_per_token() for g in plan_groups(requests)) * item
    state = sum(math.prod(s.shape) * torch.empty((), dtype=s.dtype).element_size() for _r, s in requests if s is not None)
    return {"weight_bytes": int(weights), "kv_bytes_per_token": int(per_token), "state_bytes_per_request": int(state)}


@dataclass
class CachePlan:
    page_size: int
    num_pages: int
    num_state_slots: int


def plan_cache(model, page_size: int, num_pages: int | None, activation_reserve: float, num_state_slots: int,
               dtype: torch.dtype) -> CachePlan:
    """Pool size: given, or what fits into the free device memory after the
    reserve (python/stride_worker/worker.py:182-225)."""
    if num_pages is None:
        from ..cache import plan_groups
        item = torch.empty((), dtype=dtype).element_size()
        per_page = sum(g.bytes_per_page(page_size, item) for g in plan_groups(model.cache_requests()))
        free_bytes, _total = torch.cuda.mem_get_info(model.rt.device)
        usable = int(free_bytes * (1.0 - activation_reserve))
        num_pages = usable // max(per_page, 1) if per_page else 1
        if num_pages < 1:
            raise RuntimeError(f"no room for even one KV page: {free_bytes / 2**30:.1f} GiB free, "
                               f"{per_page / 2**20:.1f} MiB needed per page")
    return CachePlan(page_size, int(num_pages), num_state_slots)


def attach_cache(model, plan: CachePlan, prefix_caching: bool = True):
    """Allocates the device cache for ``model`` and the host manager that names its pages."""
    device_cache = DeviceCache(model, plan.page_size, plan.num_pages, plan.num_state_slots, model.rt.dtype, model.rt.device)
    has_state = bool(device_cache.states)
    manager = CacheManager(plan.page_size, device_cache.group_configs(), plan.num_state_slots,
                           prefix_caching and not has_state)
    return device_cache, manager
