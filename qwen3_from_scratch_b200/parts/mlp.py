"""SwiGLU feed-forward: y = (up(x) * silu(gate(x))) W_down^T, no biases.

Reference: models/feedback.py:14-34.  gate_proj and up_proj are merged into one
[2I, H] weight at load (gate rows first), so one product feeds the gate kernel.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from ..registry import register_part
from .base import FeedForward, Runtime, WeightSpec
from .linear import Linear


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, name: str, hidden_size: int, intermediate_size: int):
        super().__init__(name)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)

    def weight_specs(self) -> List[WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [WeightSpec(f"{self.name}.gate_proj.weight", (i, h)),
                WeightSpec(f"{self.name}.up_proj.weight", (i, h)),
                WeightSpec(f"{self.name}.down_proj.weight", (h, i))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        gate = weights.pop(f"{self.name}.gate_proj.weight")
        up = weights.pop(f"{self.name}.up_proj.weight")
        dtype = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        merged = torch.cat([gate.to(dtype), up.to(dtype)], dim=0)
        del gate, up
        self.gate_up = Linear(merged, rt, tag="ffn.gate_up")
        self.down = Linear(weights.pop(f"{self.name}.down_proj.weight"), rt, tag="ffn.down")
        self._act = rt.shared("ffn.act", rt.max_tokens, self.intermediate_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gu = self.gate_up(x)
        act = self._act[: x.shape[0]]
        ops.swiglu(gu, act)
        return self.down(act)
