"""Reading and writing the safetensors container without any helper package.

A file is an 8-byte little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), and the raw little-endian tensor bytes.
Shards are found as the reference finds them
(python/stride_worker/model.py:60-76): the ``weight_map`` of
``model.safetensors.index.json`` if that file exists, else every
``*.safetensors`` file of the folder in sorted order.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightFileError(ValueError):
    pass


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: torch.dtype
    shape: tuple
    file: str
    begin: int      # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """One memory-mapped shard. Tensors are views of the mapping until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"cannot open {path}: {e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightFileError(f"{path} is too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) if isinstance(header, dict) else {}
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        base = 8 + hlen
        self.records: dict[str, TensorRecord] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise WeightFileError(f"{path}: malformed entry for tensor {name!r}") from None
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * torch.empty((), dtype=dtype).element_size() or base + end > size or begin < 0:
                raise WeightFileError(f"{path}: tensor {name!r} has offsets [{begin}, {end}) that do not match "
                                      f"its shape {shape} and dtype, or leave the file")
            self.records[name] = TensorRecord(name, dtype, shape, path, base + begin, base + end)

    def read(self, name: str) -> torch.Tensor:
        r = self.records[name]
        if r.end == r.begin:
            return torch.empty(r.shape, dtype=r.dtype)
        count = (r.end - r.begin) // torch.empty((), dtype=r.dtype).element_size()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only; nothing writes through the view
            flat = torch.frombuffer(self._map, dtype=r.dtype, count=count, offset=r.begin)
        return flat.view(r.shape)


def find_shards(model_dir: str) -> list[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            try:
                mapping = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise WeightFileError(f"{index} has no weight_map") from None
        names = sorted(set(mapping.values()))
    else:
        names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors")) if os.path.isdir(model_dir) else []
    if not names:
        raise FileNotFoundError(f"no .safetensors weights under {model_dir}")
    return [os.path.join(model_dir, n) for n in names]


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    """Writes ``tensors`` (name -> CPU tensor) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = sorted(tensors)
    for name in ordered:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightFileError(f"tensor {name!r} has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in ordered:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
