"""Matrix product y = x W^T with a weight in the checkpoint's [out, in] layout.

bfloat16: the product is a library call (cuBLAS through ``torch.mm``), as in the
reference's engine, whose projections are ``nn.Linear`` (models/self_attn.py:358-386,
models/feedback.py:28-34).  float32: the engine's own FFMA kernel, never a
reduced-precision mode.  A weight that was stored in float32 keeps its float32
product even in a bfloat16 run.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class Linear:
    """Not a registered part of its own: mixers and feed-forwards own their projections."""

    def __init__(self, weight: torch.Tensor, compute_dtype: torch.dtype, max_rows: Optional[int],
                 out_dtype: Optional[torch.dtype] = None):
        """``max_rows``: rows of the reused output buffer; None allocates the output at every call
        (for the head, whose row count is what the caller wants and whose rows are a vocabulary wide)."""
        if weight.dim() != 2:
            raise ValueError(f"a projection weight is 2-D, got {tuple(weight.shape)}")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.compute_dtype = compute_dtype
        self.out_dtype = out_dtype or compute_dtype
        self.full_precision = weight.dtype == torch.float32
        self.max_rows = max_rows
        self._out = self._out32 = None
        if max_rows is not None:
            self._out = torch.empty(max_rows, self.out_features, dtype=self.out_dtype, device=weight.device)
            if self.full_precision:
                self._out32 = self._out if self.out_dtype == torch.float32 else torch.empty(
                    max_rows, self.out_features, dtype=torch.float32, device=weight.device)
        self._weight_t = self.weight.t()

    def _buffer(self, which: str, rows: int, dtype: torch.dtype) -> torch.Tensor:
        buf = getattr(self, which)
        if buf is None:
            return torch.empty(rows, self.out_features, dtype=dtype, device=self.weight.device)
        return buf[:rows]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
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
