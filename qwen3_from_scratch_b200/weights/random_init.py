"""Random weights: writes a model folder (config.json + model.safetensors) from a configuration
and a seed, so that the real loader is what every test and benchmark goes through.

Matrices and embeddings are N(0, 0.02), norm weights 1 + N(0, 0.1).  Every tensor has a
generator of its own, seeded from (seed, tensor name), so a tensor's values do not depend on
which other tensors the model has or on the order they are written in.

``random_weights_on_device`` fills a model of any size straight on the GPU (same distributions,
a CUDA generator per tensor): a model of tens of gigabytes then needs no file of that size.  Its
values are not those of the folder writer's (another generator).
"""

from __future__ import annotations

import hashlib
import os
from typing import Dict, Optional, Sequence

import torch

from ..config.model_config import ModelConfig
from ..parts.base import WeightSpec
from ..registry import build_model_spec
from .safetensors_io import SafetensorsWriter
from .specs import model_weight_specs

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype) -> torch.Tensor:
    g = _generator(seed, spec.name)
    if spec.kind == "index":
        return torch.zeros(spec.shape, dtype=torch.int32)
    if spec.init == "normal":
        t = torch.randn(spec.shape, generator=g, dtype=torch.float32) * 0.02
    elif spec.init == "one_plus_normal":
        t = 1.0 + torch.randn(spec.shape, generator=g, dtype=torch.float32) * 0.1
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=torch.float32)
    else:
        raise ValueError(f"tensor '{spec.name}': unknown init '{spec.init}'")
    return t.to(dtype)


def write_random_model(folder: str, config: ModelConfig, seed: int, dtype: str = "bfloat16",
                       float32_tensors: Optional[Dict[str, bool]] = None) -> str:
    """Creates ``folder`` with config.json and model.safetensors.  ``dtype``: how tensors are
    stored; names in ``float32_tensors`` are stored in float32 regardless."""
    if dtype not in _STORE:
        raise ValueError(f"dtype must be one of {sorted(_STORE)}, got '{dtype}'")
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    specs = model_weight_specs(build_model_spec(config))
    keep32 = set(float32_tensors or ())

    def stored(spec: WeightSpec) -> torch.dtype:
        if spec.kind == "index":
            return torch.int32
        return torch.float32 if spec.name in keep32 else _STORE[dtype]

    decl = [(s.name, tuple(s.shape), stored(s)) for s in specs]
    path = os.path.join(folder, "model.safetensors")
    with SafetensorsWriter(path, decl, metadata={"format": "pt", "seed": seed}) as w:
        for s in specs:
            w.write(s.name, random_tensor(s, seed, stored(s)))
    return folder


def random_weights_on_device(specs: Sequence[WeightSpec], seed: int, device, compute_dtype: torch.dtype
                             ) -> Dict[str, torch.Tensor]:
    """Every tensor the specs name, drawn on ``device``: what ``load_weights`` would return for a folder
    stored in bfloat16 (matrices in ``compute_dtype``, vectors float32, integer tables int32)."""
    device = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    g = torch.Generator(device=device)
    for spec in specs:
        digest = hashlib.sha256(f"{seed}:{spec.name}".encode()).digest()
        g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
        if spec.kind == "index":
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        dtype = torch.float32 if spec.kind == "vector" else compute_dtype
        t = torch.empty(spec.shape, dtype=dtype, device=device)
        if spec.init == "normal":
            t.normal_(0.0, 0.02, generator=g)
        elif spec.init == "one_plus_normal":
            t.normal_(1.0, 0.1, generator=g)
        elif spec.init == "zeros":
            t.zero_()
        else:
            raise ValueError(f"tensor '{spec.name}': unknown init '{spec.init}'")
        out[spec.name] = t
    return out
