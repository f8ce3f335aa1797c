"""Weights from a model folder, by tensor name, onto the device.

The reference loads every tensor of every shard into a CPU dict and lets a missing name
surface as a bare KeyError, never checks for leftovers and never checks dtypes
(models/parameter_loader.py:8-48, models/common.py:4-9).  Here the folder is checked
against the model's list of ``WeightSpec`` before anything is copied, and everything
that is wrong is reported in one error: missing tensors, unexpected tensors, wrong
shapes, unusable dtypes.

What each tensor becomes (``WeightSpec.kind``):
  matrix  bfloat16 stays bfloat16; float32 stays float32 (its product then runs in
          float32); float16 is widened to float32.  In a float32 run all become float32.
  vector  float32 on the device, whatever it was stored as.
  index   int32.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Sequence

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, model_files

_FLOAT = ("F32", "BF16", "F16", "F64")
_INT = ("I64", "I32", "I16", "I8", "U8")


class WeightsError(ValueError):
    """The model folder does not hold what the model needs.  ``missing``, ``unexpected``,
    ``wrong_shape`` and ``wrong_dtype`` carry the details that the message lists."""

    def __init__(self, folder, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), other=()):
        self.folder = folder
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.other = list(other)
        lines = [f"weights in {folder} do not match the model:"]
        if self.other:
            lines += [f"  {x}" for x in self.other]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} is {list(got)}, the model needs {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n} is {got}, the model needs {want}" for n, got, want in self.wrong_dtype))
        super().__init__("\n".join(lines))


def _target_dtype(spec: WeightSpec, stored: str, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "index":
        return torch.int32
    if spec.kind == "vector" or compute_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16 if stored == "BF16" else torch.float32


def load_weights(folder: str, specs: Sequence[WeightSpec], *, device, compute_dtype: torch.dtype,
                 ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """All tensors the specs name, on ``device``.  Raises one ``WeightsError`` for everything wrong."""
    try:
        files = [SafetensorsFile(p) for p in model_files(folder)]
    except (SafetensorsError, OSError) as e:
        raise WeightsError(folder, other=[str(e)]) from None
    try:
        where = {}
        other: List[str] = []
        for f in files:
            for name in f.entries:
                if name in where:
                    other.append(f"tensor '{name}' is in both {where[name].path} and {f.path}")
                where[name] = f
        wanted = {s.name: s for s in specs}
        if len(wanted) != len(specs):
            raise ValueError("the model names a tensor twice")
        ignorable = set(ignorable)
        missing = [n for n in wanted if n not in where]
        unexpected = sorted(n for n in where if n not in wanted and n not in ignorable)
        wrong_shape, wrong_dtype = [], []
        for name, spec in wanted.items():
            if name not in where:
                continue
            e = where[name].entries[name]
            if tuple(e.shape) != tuple(spec.shape):
                wrong_shape.append((name, tuple(e.shape), tuple(spec.shape)))
            allowed = _INT if spec.kind == "index" else _FLOAT
            if e.dtype not in allowed:
                wrong_dtype.append((name, e.dtype, "an integer type" if spec.kind == "index" else "a float type"))
        if missing or unexpected or wrong_shape or wrong_dtype or other:
            raise WeightsError(folder, missing, unexpected, wrong_shape, wrong_dtype, other)
        out: Dict[str, torch.Tensor] = {}
        for name, spec in wanted.items():
            f = where[name]
            stored = f.entries[name].dtype
            host = f.get(name)
            out[name] = host.to(device=device, dtype=_target_dtype(spec, stored, compute_dtype)).contiguous()
            del host
        return out
    finally:
        for f in files:
            f.close()
