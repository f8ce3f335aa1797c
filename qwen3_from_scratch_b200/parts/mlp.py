"""SwiGLU feed-forward: y = (up(x) * silu(gate(x))) W_down^T, no biases.

Reference: models/feedback.py:14-34.  gate_proj and up_proj are merged into one
[2I, H] weight at load (gate rows first), so one product feeds the gate kernel.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from ..registry import register_part
from .base import FeedForward, Runtime, StreamNorm, WeightSpec
from .linear import Linear


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    graph_capturable = True

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
        h, i = self.hidden_size, self.intermediate_size
        # bfloat16: gate and up rows alternate in blocks of eight, so that the decode kernel has a
        # gate value and its up value in one thread and applies the activation before storing
        self.blocks_of_eight = dtype == torch.bfloat16 and i % 8 == 0
        if self.blocks_of_eight:
            merged = torch.cat([gate.view(i // 8, 8, h), up.view(i // 8, 8, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            merged = torch.cat([gate.to(dtype), up.to(dtype)], dim=0)
        del gate, up
        self.gate_up = Linear(merged, rt, tag="ffn.gate_up")
        self.down = Linear(weights.pop(f"{self.name}.down_proj.weight"), rt, tag="ffn.down")
        self._act = rt.shared("ffn.act", rt.max_tokens, self.intermediate_size)

    fuses_stream = True

    def can_fuse_stream(self, rows: int) -> bool:
        return self.blocks_of_eight and self.gate_up.takes_stream_norm(rows) and self.down.can_add_into_stream(rows)

    def forward(self, x, into_stream=None, next_norm_weight=None):
        act = self._act[: x.shape[0]]
        rows = x.shape[0]
        if isinstance(x, StreamNorm):
            # decoding without norm kernels: the norm is applied inside the gate/up product
            ops.gemm_skinny_normed(x.scaled, x.sumsq, x.parts, x.eps, self.gate_up.weight, act, swiglu_blocks=True)
        elif self.blocks_of_eight and ops.gemm_skinny_takes(rows, self.gate_up.weight):
            # decoding: stream the weight once, activation applied before the store
            ops.gemm_skinny(x, self.gate_up.weight, act, swiglu_blocks=True)
        elif (self.blocks_of_eight and ops.gemm_tc_swiglu_pays(rows, self.gate_up.weight)
              and ops.gemm_tc_takes(x, self.gate_up.weight)):
            # prompt portions: the engine's tcgen05 product with the activation in its epilogue, so the
            # [T, 2I] gate/up product never goes to memory
            ops.gemm_tc(x, self.gate_up.weight, act, self.rt.status, swiglu_blocks=True,
                        pair=ops.gemm_tc_swiglu_pays(rows, self.gate_up.weight) == "pair")
        else:
            ops.swiglu(self.gate_up(x), act, interleave8=self.blocks_of_eight)
        if into_stream is not None:
            return self.down.into_stream(act, into_stream, next_norm_weight)
        return self.down(act)
