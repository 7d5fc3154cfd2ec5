"""Where tensors come from: a model folder of safetensors shards, a dictionary in
memory, or a seeded random generator. All give tensors by checkpoint name."""

from __future__ import annotations

import torch

from .safetensors_io import SafetensorsFile, find_shards


class WeightSource:
    def names(self) -> list[str]:
        raise NotImplementedError

    def describe(self, name: str) -> tuple:
        """(shape, dtype) as stored."""
        raise NotImplementedError

    def read(self, name: str) -> torch.Tensor:
        """The stored tensor on the CPU (possibly a view of a file mapping)."""
        raise NotImplementedError


class SafetensorsSource(WeightSource):
    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files = [SafetensorsFile(p) for p in find_shards(model_dir)]
        self._where = {}
        for f in self._files:
            for name in f.records:
                self._where[name] = f

    def names(self):
        return list(self._where)

    def describe(self, name):
        r = self._where[name].records[name]
        return r.shape, r.dtype

    def read(self, name):
        return self._where[name].read(name)


class DictSource(WeightSource):
    def __init__(self, state: dict):
        self._state = state

    def names(self):
        return list(self._state)

    def describe(self, name):
        t = self._state[name]
        return tuple(t.shape), t.dtype

    def read(self, name):
        return self._state[name]


class RandomSource(WeightSource):
    """Seeded random weights for a set of declared tensors: matrices N(0, std),
    vectors (norm weights) ``1 + N(0, vector_jitter)``, biases N(0, std).

    Each tensor has its own generator, seeded from the seed and the tensor's
    name, so a value does not depend on the order of reads. ``device`` chooses
    where numbers are drawn: "cpu" gives the values that ``write_random_model``
    stores; "cuda" draws on the GPU (another stream of numbers, far faster for
    large shapes).
    """

    def __init__(self, declared: dict, seed: int, std: float = 0.02, vector_jitter: float = 0.0,
                 stored_dtype: torch.dtype = torch.bfloat16, device: str = "cpu"):
        self._declared = declared
        self.seed = int(seed)
        self.std = std
        self.vector_jitter = vector_jitter
        self.stored_dtype = stored_dtype
        self.device = device

    def names(self):
        return list(self._declared)

    def describe(self, name):
        return tuple(self._declared[name].shape), self.stored_dtype

    def _generator(self, name: str) -> torch.Generator:
        h = 0xCBF29CE484222325
        for b in name.encode():
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        g = torch.Generator(device=self.device)
        g.manual_seed((h ^ (self.seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF)
        return g

    def read(self, name):
        decl = self._declared[name]
        g = self._generator(name)
        x = torch.randn(tuple(decl.shape), generator=g, dtype=torch.float32, device=self.device)
        if decl.role == "vector":
            x = 1.0 + x * self.vector_jitter
        else:
            x = x * self.std
        return x.to(self.stored_dtype)
