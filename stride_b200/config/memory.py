"""Capacity planning for one GPU: do the weights fit, and how much cache is left.

Weights, the working set of a step and the cache share the device's memory; the
cache is what the other two leave. The subtraction is done here, before anything
is loaded, so that a model that cannot run is refused with its numbers instead
of an out-of-memory error in the middle of a request
(crates/stride-model/src/memory.rs:67-121, without its per-rank split: one GPU).
``plan_cache`` in the engine does the same from the free memory it finds at run
time; this is the arithmetic alone, needs no GPU, and backs the ``plan`` command.
"""

from __future__ import annotations

from dataclasses import dataclass

GIB = float(1 << 30)
B200_MEMORY_BYTES = 183_359 * (1 << 20)       # what the driver reports for a B200 (180 GB HBM3e)
ITEMSIZE = {"bfloat16": 2, "float32": 4}


class PlanError(ValueError):
    pass


@dataclass(frozen=True)
class MemoryPlan:
    model: str
    dtype: str
    block_size: int
    memory_bytes: int
    weight_bytes: int
    activation_reserve_bytes: int
    kv_bytes: int
    kv_bytes_per_token: int
    num_blocks: int

    @property
    def total_kv_tokens(self) -> int:
        return self.num_blocks * self.block_size

    def max_context(self) -> int:
        """The longest single request the cache can hold."""
        return self.total_kv_tokens

    def concurrent_sequences(self, context: int) -> int:
        """Requests of ``context`` tokens that fit at once, without prefix sharing (memory.rs:127-133)."""
        if context <= 0:
            return 0
        return self.num_blocks // max(1, -(-context // self.block_size))

    def describe(self) -> str:
        return "\n".join([
            f"{self.model} in {self.dtype} on {self.memory_bytes / GIB:.1f} GiB",
            f"  weights             {self.weight_bytes / GIB:9.2f} GiB",
            f"  activation reserve  {self.activation_reserve_bytes / GIB:9.2f} GiB",
            f"  cache               {self.kv_bytes / GIB:9.2f} GiB  ({self.kv_bytes_per_token} bytes a token)",
            f"  pages of {self.block_size:<4}       {self.num_blocks:9d}      ({self.total_kv_tokens} tokens)",
        ])


def plan_memory(config, dtype: str = "bfloat16", memory_bytes: int = B200_MEMORY_BYTES, block_size: int = 16,
                activation_fraction: float = 0.15, name: str | None = None, max_requests: int = 256) -> MemoryPlan:
    """``config``: the typed configuration of any registered architecture. Its sizes are taken from the model's
    own parts (the tensors they declare, what their mixers keep per token and per request), not from arithmetic
    on the configuration class. ``activation_fraction`` of what the weights leave is held back for activations,
    workspace and fragmentation (the worker's ``--activation-reserve``, python/stride_worker/worker.py:182-225);
    state of fixed size is set aside for ``max_requests`` requests. Raises ``PlanError`` when the weights do not
    fit or not even one page is left."""
    if dtype not in ITEMSIZE:
        raise PlanError(f"dtype must be one of {sorted(ITEMSIZE)}, got {dtype!r}")
    if block_size <= 0:
        raise PlanError("block_size must be positive")
    if not 0.0 <= activation_fraction < 1.0:
        raise PlanError("activation_fraction must be in [0, 1)")
    from ..engine.loading import footprint      # the parts live above this package; asked for only when a plan is made
    sizes = footprint(config, dtype)
    name = name or getattr(config, "name", "model")
    weight_bytes = sizes["weight_bytes"] + sizes["state_bytes_per_request"] * max_requests
    if weight_bytes >= memory_bytes:
        raise PlanError(f"{name}: the weights need {weight_bytes / GIB:.1f} GiB in {dtype} but the device has "
                        f"{memory_bytes / GIB:.1f} GiB")
    after_weights = memory_bytes - weight_bytes
    reserve = int(after_weights * activation_fraction)
    kv_bytes = after_weights - reserve
    per_token = max(1, sizes["kv_bytes_per_token"])
    num_blocks = kv_bytes // (per_token * block_size)
    if num_blocks == 0:
        raise PlanError(f"{name}: {kv_bytes / GIB:.2f} GiB are left for the cache after weights and activations, less than "
                        f"the {per_token * block_size / GIB:.4f} GiB of one page of {block_size} tokens")
    return MemoryPlan(model=name, dtype=dtype, block_size=block_size, memory_bytes=int(memory_bytes), weight_bytes=int(weight_bytes),
                      activation_reserve_bytes=reserve, kv_bytes=int(kv_bytes), kv_bytes_per_token=int(per_token),
                      num_blocks=int(num_blocks))
