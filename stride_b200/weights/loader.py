"""Loading weights by tensor name, with one error for everything that is wrong.

A model declares the tensors it reads: name, shape and a role. The loader
compares that with what the source holds and raises a single
``WeightMismatchError`` that lists missing tensors, unexpected tensors and
tensors of the wrong shape (the reference raises on the first missing name
only, python/stride_worker/model.py:136-143, and checks no shape).

Element types on the device:
  * role ``matrix`` (operands of matrix products, the embedding table): the
    compute dtype, bfloat16 or float32, whatever the file holds
    (python/stride_worker/model.py:120-121,143);
  * role ``vector`` (norm weights, biases): float32, which keeps a tensor stored
    in 32-bit as it is and widens a 16-bit one without loss; the kernels read
    these in float32;
  * role ``table`` (integer tables): int32.
"""

from __future__ import annotations

import fnmatch
from dataclasses import dataclass

import torch

from .sources import WeightSource


@dataclass(frozen=True)
class TensorDecl:
    shape: tuple
    role: str = "matrix"        # matrix | vector | table
    optional: bool = False


class WeightMismatchError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, wrong_kind):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_kind = sorted(wrong_kind)
        lines = ["the checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " +
                         ", ".join(f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong element kinds ({len(self.wrong_kind)}): " +
                         ", ".join(f"{n} is {got}, expected {want}" for n, got, want in self.wrong_kind))
        super().__init__("\n".join(lines))


def target_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute_dtype
    if role == "vector":
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown tensor role {role!r}")


def check_source(source: WeightSource, declared: dict, ignorable: tuple = ()) -> None:
    have = set(source.names())
    missing = [n for n, d in declared.items() if n not in have and not d.optional]
    unexpected = [n for n in have if n not in declared and not any(fnmatch.fnmatch(n, pat) for pat in ignorable)]
    wrong_shape, wrong_kind = [], []
    for n, d in declared.items():
        if n not in have:
            continue
        shape, dtype = source.describe(n)
        if tuple(shape) != tuple(d.shape):
            wrong_shape.append((n, tuple(shape), tuple(d.shape)))
        is_float = dtype.is_floating_point
        if (d.role == "table") == is_float:
            wrong_kind.append((n, str(dtype), "an integer type" if d.role == "table" else "a floating-point type"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightMismatchError(missing, unexpected, wrong_shape, wrong_kind)


def load_weights(source: WeightSource, declared: dict, compute_dtype: torch.dtype, device, ignorable: tuple = (),
                 checked: bool = False) -> dict:
    """Checks the source against the declarations (unless the caller has checked the whole model already and
    now loads it part by part), then moves every declared tensor to ``device`` in its target dtype. Returns
    name -> tensor."""
    if not checked:
        check_source(source, declared, ignorable)
    have = set(source.names())
    out = {}
    for name, decl in declared.items():
        if name not in have:
            continue
        t = source.read(name)
        out[name] = t.to(device=device, dtype=target_dtype(decl.role, compute_dtype)).contiguous()
    return out
