"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, statistics in float32.

Reference: models/norm.py:11-22 (weight multiplies directly, eps from the configuration),
csrc/rms_norm/rms_norm.cpp:13-31.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import Norm, Runtime, StreamNorm, StreamStats, WeightSpec


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    graph_capturable = True

    def __init__(self, name: str, dim: int, eps: float):
        super().__init__(name)
        self.dim, self.eps = int(dim), float(eps)

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(f"{self.name}.weight", (self.dim,), kind="vector", init="one_plus_normal")]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight = weights[f"{self.name}.weight"]
        self._out = rt.shared("normed", rt.max_tokens, self.dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        ops.rmsnorm(x, self.weight, out, self.eps)
        return out

    def add_norm(self, stream: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = self._out[: stream.shape[0]]
        ops.add_rmsnorm(stream, delta, self.weight, out, self.eps)
        return out

    def lazy(self, stream: torch.Tensor, stats: StreamStats) -> Optional[StreamNorm]:
        """This norm of the stream for a projection that applies it itself, if the projection that last
        added into the stream prepared the stream for this norm's weight; else None."""
        if stats is None or stats.scaled is None or stats.scaled_for is not self.weight:
            return None
        return StreamNorm(stream, self.weight, self.eps, stats.sumsq, stats.parts, stats.scaled)

    def norm_rows(self, stream: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.numel(), self.dim, dtype=self.rt.dtype, device=stream.device)
        ops.add_rmsnorm_rows(stream, delta, self.weight, rows, out, self.eps)
        return out
