"""Grouped-query attention over a paged cache, with optional per-head RMSNorm of q and k,
an optional position encoding, and an optional sliding window.

Reference: models/self_attn.py:300-386 (packed [T, hidden] input, merged QKV, head norm then
rotation, keys/values written to pages, causal attention over the cache, output projection),
models/attn.py:388-499 (scale = head_dim^-0.5, q head h reads kv head h // (Hq / Hkv)).
The window (a query at position p reads keys p - window < n <= p) is what config.json's
``sliding_window`` asks of a layer; the reference itself never reads that key.
In a step where every row brings one token the decode attention kernel does the head norm, the
rotation and the page write itself, from the raw QKV projection.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import create_part, register_part
from .base import KVCacheSpec, Mixer, PartSpec, Runtime, StepContext, WeightSpec
from .linear import Linear


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    graph_capturable = True

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm_eps: Optional[float] = None, position: Optional[PartSpec] = None,
                 window: Optional[int] = None):
        super().__init__(name)
        self.hidden_size = int(hidden_size)
        self.num_heads, self.num_kv_heads, self.head_dim = int(num_heads), int(num_kv_heads), int(head_dim)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads are not a multiple of {self.num_kv_heads} kv heads")
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.position = create_part("position", position, name=f"{name}.position") if position else None
        self.scale = float(self.head_dim) ** -0.5

    # ------------------------------------------------------------------ declarations
    def weight_specs(self) -> List[WeightSpec]:
        h, d = self.hidden_size, self.head_dim
        specs = [WeightSpec(f"{self.name}.q_proj.weight", (self.num_heads * d, h)),
                 WeightSpec(f"{self.name}.k_proj.weight", (self.num_kv_heads * d, h)),
                 WeightSpec(f"{self.name}.v_proj.weight", (self.num_kv_heads * d, h)),
                 WeightSpec(f"{self.name}.o_proj.weight", (h, self.num_heads * d))]
        if self.qk_norm_eps is not None:
            specs += [WeightSpec(f"{self.name}.q_norm.weight", (d,), kind="vector", init="one_plus_normal"),
                      WeightSpec(f"{self.name}.k_norm.weight", (d,), kind="vector", init="one_plus_normal")]
        if self.position is not None:
            specs += self.position.weight_specs()
        return specs

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    # ------------------------------------------------------------------ device side
    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        q = weights.pop(f"{self.name}.q_proj.weight")
        k = weights.pop(f"{self.name}.k_proj.weight")
        v = weights.pop(f"{self.name}.v_proj.weight")
        dtype = torch.float32 if torch.float32 in (q.dtype, k.dtype, v.dtype) else q.dtype
        merged = torch.cat([q.to(dtype), k.to(dtype), v.to(dtype)], dim=0)  # rows ordered q, k, v
        del q, k, v
        self.qkv = Linear(merged, rt, tag="attn.qkv")
        self.o_proj = Linear(weights.pop(f"{self.name}.o_proj.weight"), rt, tag="attn.o_proj")
        self.q_norm_weight = self.k_norm_weight = None
        if self.qk_norm_eps is not None:
            self.q_norm_weight = weights[f"{self.name}.q_norm.weight"]
            self.k_norm_weight = weights[f"{self.name}.k_norm.weight"]
        if self.position is not None:
            self.position.setup(rt, weights)
        self._q = rt.shared("attn.q", rt.max_tokens, self.num_heads, self.head_dim)
        self._o = rt.shared("attn.o", rt.max_tokens, self.num_heads, self.head_dim)
        self._partial = None
        if ops.fast_attention_takes(rt.dtype, self.num_heads, self.num_kv_heads, self.head_dim):
            self._partial = rt.shared("attn.partial", ops.decode_partial_numel(rt.max_seqs, self.num_heads,
                                                                               self.head_dim), dtype=torch.float32)

    fuses_stream = True

    def can_fuse_stream(self, rows: int) -> bool:
        return self.qkv.takes_stream_norm(rows) and self.o_proj.can_add_into_stream(rows)

    def forward(self, x, ctx: StepContext, cache_id: Optional[int], write_cache: bool, into_stream=None,
                next_norm_weight=None):
        """``x``: the normed activations, or a ``StreamNorm`` that the QKV product applies itself.
        ``into_stream``: the output projection adds into this stream and its ``StreamStats`` are returned
        (with the rows times ``next_norm_weight`` if that is given)."""
        T = x.shape[0]
        hq, hkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        k_pages, v_pages, table = ctx.kv(cache_id)
        q = self._q[:T]
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        fused = self.position.fused_rotary() if self.position is not None else None
        out = self._o[:T]
        whole_rotation = fused is None or fused[1] == d
        if ((self.position is None or fused is not None) and whole_rotation
                and ops.decode_takes_raw_qkv(self.rt.dtype, hq, hkv, d, k_pages.shape[2], T, ctx.num_seqs, ctx.num_decode)):
            # every row decodes: the attention kernel norms and rotates its own query and the new key itself
            # (the step's angles are made before the projection, so that the kernel may fetch them early)
            cos_sin = self.position.step_table(ctx) if fused is not None else None
            qkv = self.qkv(x)
            raw = (qkv, self.q_norm_weight, self.k_norm_weight, eps, cos_sin, write_cache)
            self.attend(q, k_pages, v_pages, table, ctx, out, raw_qkv=raw)
            if into_stream is not None:
                return self.o_proj.into_stream(out.view(T, hq * d), into_stream, next_norm_weight)
            return self.o_proj(out.view(T, hq * d))
        if ((self.position is None or fused is not None) and torch.is_tensor(x)
                and ops.gemm_tc_qkv_takes(T, x, self.qkv.weight, d, fused[1] if fused is not None else 0)
                and ops.gemm_tc_qkv_pays(T, self.qkv.weight)):
            # a prompt portion: the projection's own epilogue norms, rotates and writes the pages
            cos_sin = self.position.step_table(ctx) if fused is not None else None
            ops.gemm_tc_qkv(x, self.qkv.weight, q, k_pages, v_pages, self.q_norm_weight, self.k_norm_weight, eps,
                            cos_sin, ctx.positions, ctx.tok_seq, table, hq, hkv, d, write_cache, self.rt.status,
                            pair=ops.gemm_tc_qkv_pays(T, self.qkv.weight) == "pair")
            self.attend(q, k_pages, v_pages, table, ctx, out)
            if into_stream is not None:
                return self.o_proj.into_stream(out.view(T, hq * d), into_stream, next_norm_weight)
            return self.o_proj(out.view(T, hq * d))
        qkv = self.qkv(x)
        if self.position is None or fused is not None:
            inv_freq, rotary_dim = fused if fused is not None else (None, 0)
            cos_sin = self.position.step_table(ctx) if fused is not None else None
            ops.qkv_post(qkv, q, k_pages, v_pages, self.q_norm_weight, self.k_norm_weight, eps, inv_freq,
                         rotary_dim, ctx.positions, ctx.tok_seq, table, hq, hkv, d, write_cache, self.rt.status,
                         cos_sin=cos_sin)
        else:
            # a position encoding the kernel does not know: norm, encode, then scatter, as separate steps
            heads = qkv.view(T, hq + 2 * hkv, d)
            qh = heads[:, :hq].contiguous()
            kh = heads[:, hq:hq + hkv].contiguous()
            if self.qk_norm_eps is not None:
                qn, kn = torch.empty_like(qh), torch.empty_like(kh)
                ops.rmsnorm(qh, self.q_norm_weight, qn, eps)
                ops.rmsnorm(kh, self.k_norm_weight, kn, eps)
                qh, kh = qn, kn
            heads[:, :hq].copy_(self.position.apply(qh, ctx.positions))
            heads[:, hq:hq + hkv].copy_(self.position.apply(kh, ctx.positions))
            ops.qkv_post(qkv, q, k_pages, v_pages, None, None, 0.0, None, 0, ctx.positions, ctx.tok_seq, table,
                         hq, hkv, d, write_cache, self.rt.status)
        self.attend(q, k_pages, v_pages, table, ctx, out)
        if into_stream is not None:
            return self.o_proj.into_stream(out.view(T, hq * d), into_stream, next_norm_weight)
        return self.o_proj(out.view(T, hq * d))

    def attend(self, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
               ctx: StepContext, out: torch.Tensor, raw_qkv=None) -> None:
        """Causal attention of this step's queries over the pages (keys of this step included)."""
        ops.paged_attention(q, k_pages, v_pages, out, ctx.q_start, ctx.kv_len, ctx.tok_seq, table, ctx.num_seqs,
                            ctx.num_decode, ctx.max_q_len, ctx.max_kv_len, self.scale, self.window or 0,
                            self.rt.status, self._partial, raw_qkv=raw_qkv)
