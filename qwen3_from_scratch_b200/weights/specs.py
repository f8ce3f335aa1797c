"""The list of tensors a model specification needs, without touching a device."""

from __future__ import annotations

from typing import List

from ..parts.base import ModelSpec, WeightSpec
from ..registry import create_part


def model_weight_specs(spec: ModelSpec) -> List[WeightSpec]:
    specs: List[WeightSpec] = []
    emb_name, emb = spec.embedding
    specs += create_part("embedding", emb, name=emb_name).weight_specs()
    for name, block in spec.layers:
        specs += create_part("block", block, name=name).weight_specs()
    norm_name, norm = spec.final_norm
    specs += create_part("norm", norm, name=norm_name).weight_specs()
    head_name, head = spec.head
    specs += create_part("head", head, name=head_name).weight_specs()
    seen = set()
    for s in specs:
        if s.name in seen:
            raise ValueError(f"two parts ask for the tensor '{s.name}'")
        seen.add(s.name)
    return specs
