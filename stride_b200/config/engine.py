"""Settings of the engine itself (not of a model), with the names and defaults
of the reference's command lines (python/stride_worker/worker.py:252-280:
``--dtype``, ``--block-size``, ``--num-blocks``, ``--activation-reserve``;
crates/stride-server/src/main.rs:86-107: ``--max-batch-tokens``,
``--max-batch-seqs``, ``--max-model-len``, ``--max-queued``; scheduler watermark and chunked
prefill from crates/stride-sched/src/lib.rs:31-55)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"
    block_size: int = 16                     # tokens per cache page
    num_blocks: Optional[int] = None         # pages per group; None: sized from free device memory
    activation_reserve: float = 0.15         # share of free memory kept back when sizing the pool
    max_batch_tokens: int = 2048
    max_batch_seqs: int = 256
    max_model_len: int = 8192
    max_queued: int = 1024                   # requests that may wait for admission before add_request refuses more
    watermark: float = 0.01
    chunked_prefill: bool = True
    prefix_caching: bool = True
    check_invariants: bool = False           # verify the cache manager after every step
    cuda_graphs: bool = True                 # replay decode-only steps from captured graphs
    chain_steps: bool = True                 # launch a decode step before the tokens of the one before it are read
    device_ranking: bool = True              # top-k and nucleus rows are drawn on the device too (False: on the host, from their logits)
    seed: int = 0x57219A3C11FF0042           # base of per-request fallback seeds (crates/stride-engine/src/lib.rs:85)

    def __post_init__(self):
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {self.dtype!r}")
        if self.block_size <= 0:
            raise ValueError("block_size must be positive")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        if not 0.0 <= self.activation_reserve < 1.0:
            raise ValueError("activation_reserve must be in [0, 1)")
        if self.max_batch_tokens <= 0 or self.max_batch_seqs <= 0 or self.max_model_len <= 1:
            raise ValueError("batch and length limits must be positive")
        if self.max_queued <= 0:
            raise ValueError("max_queued must be positive")

    @property
    def torch_dtype(self) -> torch.dtype:
        return DTYPES[self.dtype]
