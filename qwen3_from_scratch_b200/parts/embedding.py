"""Token embedding and the output head.

Reference: models/qwen3.py:17-19,45 (lookup, no scaling), models/qwen3.py:63-74,83-84
(head = Linear without bias, tied to the embedding table when the configuration says so).
The embedding writes the float32 residual stream; the head returns float32 logits.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import Part, Runtime, WeightSpec
from .linear import Linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_capturable = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int):
        super().__init__(name)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(f"{self.name}.weight", (self.vocab_size, self.hidden_size))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight = weights[f"{self.name}.weight"]
        self._stream = rt.shared("stream", rt.max_tokens, self.hidden_size, dtype=torch.float32)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        stream = self._stream[: token_ids.numel()]
        ops.embed(self.weight, token_ids, stream, self.rt.status)
        return stream


@register_part("head", "lm_head")
class LMHead(Part):
    graph_capturable = True

    """logits = x W^T in float32.  ``tied_to``: name of the embedding tensor it shares, or None."""

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        super().__init__(name)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tied_to = tied_to

    def weight_specs(self) -> List[WeightSpec]:
        if self.tied_to:
            return []
        return [WeightSpec(f"{self.name}.weight", (self.vocab_size, self.hidden_size))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        weight = weights[self.tied_to] if self.tied_to else weights[f"{self.name}.weight"]
        self.proj = Linear(weight, rt, out_dtype=torch.float32, reuse_output=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x)
