"""Rotary position encoding, rotate-half ("neox") pairing.

Reference: models/rotary.py:36-45 (inv_freq[j] = theta^(-2j/D), angle = position * inv_freq[j])
and models/rotary.py:13-22 (y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin on the two halves).
The angle, sine and cosine are float32 on the device.  There is no table over all positions
(``max_positions`` only bounds what a request may reach): the sines and cosines of the positions
of one step are computed once per step and read by every layer.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from ..registry import register_part
from .base import PositionEncoding, Runtime


@register_part("position", "rotary_neox")
class RotaryNeox(PositionEncoding):
    graph_capturable = True

    def __init__(self, name: str, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None):
        super().__init__(name)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        # the same float32 expression as the reference, evaluated once on the host
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(rt.device)

        self._table = rt.shared(f"rotary.table.{self.theta!r}.{self.rotary_dim}", rt.max_tokens, self.rotary_dim,
                                dtype=torch.float32)

    def fused_rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.rotary_dim

    def step_table(self, ctx) -> Optional[torch.Tensor]:
        def make():
            table = self._table[:ctx.positions.numel()]
            ops.rope_table(self.inv_freq, ctx.positions, table)
            return table
        return ctx.shared_in_step(("rotary_neox", self.theta, self.rotary_dim), make)

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        ops.rope(x, self.inv_freq, self.rotary_dim, positions, out, self.rt.status)
        return out
