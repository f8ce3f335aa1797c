"""Matrix product y = x W^T with a weight in the checkpoint's [out, in] layout.

bfloat16: with more than 16 rows the product is a library call (cuBLAS through ``torch.mm``),
as in the reference's engine, whose projections are ``nn.Linear`` (models/self_attn.py:358-386,
models/feedback.py:28-34); with up to 16 rows (decoding) it is the engine's own weight-streaming
tensor-core kernel, which can also add its result into the residual stream (``into_stream``) and
apply an RMSNorm of the stream that was never computed (``StreamNorm``).  float32: the engine's own
FFMA kernel, never a reduced-precision mode.  A weight that was stored in float32 keeps its float32
product even in a bfloat16 run.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Runtime, StreamNorm, StreamStats


class Linear:
    """Not a registered part of its own: mixers and feed-forwards own their projections."""

    def __init__(self, weight: torch.Tensor, rt: Runtime, tag: Optional[str] = None,
                 out_dtype: Optional[torch.dtype] = None, reuse_output: bool = True):
        """``tag``: role of the output buffer, shared between layers (see ``Runtime.shared``);
        None gives this projection a buffer of its own.  ``reuse_output=False`` allocates the
        output at every call (the head, whose rows are a vocabulary wide and as many as asked for)."""
        if weight.dim() != 2:
            raise ValueError(f"a projection weight is 2-D, got {tuple(weight.shape)}")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.out_dtype = out_dtype or rt.dtype
        self.full_precision = weight.dtype == torch.float32
        self.max_rows = rt.max_tokens if reuse_output else None
        self._out = self._out32 = None
        if reuse_output:
            shape = (rt.max_tokens, self.out_features)
            make = (lambda t, dt: rt.shared(f"{tag}.{t}", *shape, dtype=dt)) if tag else (
                lambda t, dt: rt.empty(*shape, dtype=dt))
            self._out = make("out", self.out_dtype)
            if self.full_precision:
                self._out32 = self._out if self.out_dtype == torch.float32 else make("out32", torch.float32)
        self._weight_t = self.weight.t()
        self._sumsq = self._scaled = None
        if not self.full_precision and rt.dtype == torch.bfloat16:
            parts = ops.sumsq_parts(self.out_features)
            rows = ops.SKINNY_MAX_ROWS
            if tag:
                self._sumsq = rt.shared(f"{tag}.sumsq", parts, ops.SUMSQ_ROWS, dtype=torch.float32)
                self._scaled = rt.shared(f"{tag}.scaled", rows, self.out_features, dtype=torch.bfloat16)
            else:
                self._sumsq = rt.empty(parts, ops.SUMSQ_ROWS, dtype=torch.float32)
                self._scaled = rt.empty(rows, self.out_features, dtype=torch.bfloat16)

    def _buffer(self, which: str, rows: int, dtype: torch.dtype) -> torch.Tensor:
        buf = getattr(self, which)
        if buf is None:
            return torch.empty(rows, self.out_features, dtype=dtype, device=self.weight.device)
        return buf[:rows]

    def takes_stream_norm(self, rows: int) -> bool:
        """Whether ``self(StreamNorm)`` works for this many rows (a bfloat16 weight, a few rows) and pays."""
        return (not self.full_precision and self.out_dtype == torch.bfloat16 and self._out is not None
                and ops.gemm_skinny_takes(rows, self.weight) and ops.gemm_skinny_normed_pays(rows, self.weight))

    def can_add_into_stream(self, rows: int) -> bool:
        return self._sumsq is not None and ops.gemm_skinny_takes(rows, self.weight)

    def into_stream(self, x: torch.Tensor, stream: torch.Tensor,
                    next_norm_weight: Optional[torch.Tensor] = None) -> StreamStats:
        """stream += x W^T for a few rows; returns what the next norm needs to know about the new rows, with
        the rows times ``next_norm_weight`` in bfloat16 if that weight is given (see StreamNorm)."""
        scaled = self._scaled[: x.shape[0]] if next_norm_weight is not None else None
        parts = ops.gemm_skinny_into_stream(x, self.weight, stream, self._sumsq, next_norm_weight, scaled)
        return StreamStats(self._sumsq, parts, scaled, next_norm_weight)

    def __call__(self, x) -> torch.Tensor:
        rows = x.shape[0]
        if isinstance(x, StreamNorm):
            if not self.takes_stream_norm(rows):
                raise ValueError("this projection does not take a norm that is not computed (see takes_stream_norm)")
            out = self._buffer("_out", rows, self.out_dtype)
            ops.gemm_skinny_normed(x.scaled, x.sumsq, x.parts, x.eps, self.weight, out)
            return out
        if self.max_rows is not None and rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the {self.max_rows} this projection was sized for")
        if self.full_precision:
            x32 = x if x.dtype == torch.float32 else x.float()
            out32 = self._buffer("_out32", rows, torch.float32)
            ops.gemm_f32_nt(x32.contiguous(), self.weight, out32)
            if self.out_dtype == torch.float32:
                return out32
            out = self._buffer("_out", rows, self.out_dtype)
            out.copy_(out32)
            return out
        if ops.gemm_skinny_takes(rows, self.weight) and x.dtype == torch.bfloat16:
            # a handful of rows: the product is a stream over the weight, done by the engine's own kernel
            out = self._buffer("_out", rows, self.out_dtype)
            ops.gemm_skinny(x, self.weight, out)
            return out
        if self.out_dtype == x.dtype:
            out = self._buffer("_out", rows, self.out_dtype)
            torch.mm(x, self._weight_t, out=out)
            return out
        wide = torch.mm(x, self._weight_t, out_dtype=self.out_dtype)
        if self._out is None:
            return wide
        out = self._out[:rows]
        out.copy_(wide)
        return out
