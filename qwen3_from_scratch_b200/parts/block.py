"""Pre-norm residual block: h = x + mixer(norm1(x)); y = h + feed_forward(norm2(h)).

Reference: models/transformer_block.py:38-46.  The residual stream is float32 and the sums are
fused into the norms: a block receives the previous sub-layer's output as ``pending`` and hands
its own feed-forward output on in the same way.  With a few rows in bfloat16 (decoding) the sums
and the norms move into the projections instead (``PreNormBlock.fuses``): the last projection of a
sub-layer adds into the stream, the first one of the next applies the norm, and no norm kernel runs.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..registry import create_part, register_part
from .base import NEXT_NORM_WEIGHT, STREAM_SUMSQ, Block, PartSpec, Runtime, StepContext, WeightSpec


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, name: str, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        n = {"norm1": "norm1", "mixer": "mixer", "norm2": "norm2", "feed_forward": "feed_forward"}
        n.update(names or {})
        self.norm1 = create_part("norm", norm1, name=f"{name}.{n['norm1']}")
        self.mixer = create_part("mixer", mixer, name=f"{name}.{n['mixer']}")
        self.norm2 = create_part("norm", norm2, name=f"{name}.{n['norm2']}")
        self.feed_forward = create_part("feed_forward", feed_forward, name=f"{name}.{n['feed_forward']}")

    @property
    def graph_capturable(self) -> bool:
        return all(p.graph_capturable for p in (self.norm1, self.mixer, self.norm2, self.feed_forward))

    def weight_specs(self) -> List[WeightSpec]:
        return (self.norm1.weight_specs() + self.mixer.weight_specs() + self.norm2.weight_specs()
                + self.feed_forward.weight_specs())

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        for part in (self.norm1, self.mixer, self.norm2, self.feed_forward):
            part.setup(rt, weights)

    keeps_stream_stats = True

    @property
    def first_norm_weight(self) -> Optional[torch.Tensor]:
        """The weight of the norm this block applies to the stream first, if the block before may prepare
        the stream for it (see StreamStats.scaled)."""
        return self.norm1.weight if hasattr(self.norm1, "lazy") else None

    def fuses(self, rows: int) -> bool:
        """A few rows (decoding) in bfloat16: the mixer's and the feed-forward's last projections add into
        the stream themselves and their first ones apply the norm, so that no norm kernel runs."""
        return (self.rt.dtype == torch.bfloat16 and hasattr(self.norm1, "lazy") and hasattr(self.norm2, "lazy")
                and getattr(self.mixer, "fuses_stream", False) and getattr(self.feed_forward, "fuses_stream", False)
                and self.mixer.can_fuse_stream(rows) and self.feed_forward.can_fuse_stream(rows))

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache_id: Optional[int], write_cache: bool) -> Optional[torch.Tensor]:
        shared = ctx.__dict__.setdefault("per_step", {})
        stats = shared.pop(STREAM_SUMSQ, None)  # of the stream as the block before left it
        if self.fuses(stream.shape[0]):
            x = self.norm1.lazy(stream, stats) if pending is None else None
            if x is None:  # the first block of a step, or one that nobody prepared the stream for
                x = self.norm1.add_norm(stream, pending)
            stats = self.mixer.forward(x, ctx, cache_id, write_cache, into_stream=stream,
                                       next_norm_weight=self.norm2.weight)
            shared[STREAM_SUMSQ] = self.feed_forward.forward(self.norm2.lazy(stream, stats), into_stream=stream,
                                                             next_norm_weight=shared.get(NEXT_NORM_WEIGHT))
            return None
        x = self.norm1.add_norm(stream, pending)
        a = self.mixer.forward(x, ctx, cache_id, write_cache)
        x = self.norm2.add_norm(stream, a)
        return self.feed_forward.forward(x)
