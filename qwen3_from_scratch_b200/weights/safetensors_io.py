"""Reading and writing safetensors files without holding a whole model in memory.

The format: 8 bytes little-endian header length N, N bytes of JSON mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the
end of the header, tensors laid out back to back), then the raw little-endian data.
The writer declares all tensors first and then streams them one by one, so a folder
larger than host memory can be produced; the reader maps the file and hands out
tensors by name.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
DTYPE_NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int  # absolute byte offsets in the file
    end: int
    path: str


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def read_header(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: truncated or not a safetensors file (header of {n} bytes, file of {size})")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    base = 8 + n
    entries: Dict[str, TensorEntry] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape = info["dtype"], tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
        if dtype not in DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has dtype {dtype}, which is not read here")
        want = _numel(shape) * torch.empty(0, dtype=DTYPES[dtype]).element_size()
        if end - begin != want:
            raise SafetensorsError(f"{path}: tensor '{name}' spans {end - begin} bytes, its shape needs {want}")
        if base + end > size:
            raise SafetensorsError(
                f"{path}: truncated: tensor '{name}' ends at byte {base + end}, the file has {size}")
        entries[name] = TensorEntry(name, dtype, shape, base + begin, base + end, path)
    return entries


class SafetensorsFile:
    """One mapped file; ``get(name)`` returns a CPU tensor that views the mapping."""

    def __init__(self, path: str):
        self.path = path
        self.entries = read_header(path)
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)

    def get(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=DTYPES[e.dtype])
        view = memoryview(self._map)[e.begin:e.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the mapping is read-only and only ever read
            return torch.frombuffer(view, dtype=DTYPES[e.dtype]).view(e.shape)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:
            pass  # tensors that still view the mapping keep it alive
        self._file.close()


def model_files(folder: str) -> List[str]:
    """``model.safetensors``, or the shards an index names, or ``model-*.safetensors`` sorted
    (the reference globs ``model.*.safetensors``: models/parameter_loader.py:26-33)."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: not an index with a 'weight_map'") from None
        files = sorted(set(weight_map.values()))
        missing = [x for x in files if not os.path.isfile(os.path.join(folder, x))]
        if missing:
            raise SafetensorsError(f"{index} names files that are not there: {', '.join(missing)}")
        return [os.path.join(folder, x) for x in files]
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    shards = sorted(x for x in os.listdir(folder) if x.startswith("model") and x.endswith(".safetensors")) \
        if os.path.isdir(folder) else []
    if not shards:
        raise SafetensorsError(f"no model.safetensors (or shards) in {folder}")
    return [os.path.join(folder, x) for x in shards]


class SafetensorsWriter:
    """Declare every tensor, then write them in the declared order."""

    def __init__(self, path: str, tensors: List[Tuple[str, Tuple[int, ...], torch.dtype]], metadata=None):
        self.path = path
        header = {}
        if metadata:
            header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
        offset = 0
        self._order = []
        for name, shape, dtype in tensors:
            if name in header:
                raise SafetensorsError(f"tensor '{name}' declared twice")
            nbytes = _numel(shape) * torch.empty(0, dtype=dtype).element_size()
            header[name] = {"dtype": DTYPE_NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
            self._order.append((name, tuple(shape), dtype, nbytes))
            offset += nbytes
        blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
        blob += b" " * ((8 - len(blob) % 8) % 8)
        self._file = open(path, "wb")
        self._file.write(struct.pack("<Q", len(blob)))
        self._file.write(blob)
        self._next = 0

    def write(self, name: str, tensor: torch.Tensor) -> None:
        if self._next >= len(self._order):
            raise SafetensorsError("more tensors written than declared")
        want_name, shape, dtype, nbytes = self._order[self._next]
        if name != want_name or tuple(tensor.shape) != shape or tensor.dtype != dtype:
            raise SafetensorsError(
                f"expected '{want_name}' {shape} {dtype} next, got '{name}' {tuple(tensor.shape)} {tensor.dtype}")
        data = tensor.detach().cpu().contiguous()
        raw = data.view(torch.uint8) if data.numel() else data
        self._file.write(raw.numpy().tobytes() if raw.numel() else b"")
        self._next += 1

    def close(self) -> None:
        if self._next != len(self._order):
            self._file.close()
            raise SafetensorsError(f"{len(self._order) - self._next} declared tensors were never written")
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            self.close()
        else:
            self._file.close()
