"""Python face of the CUDA kernels: argument checks, then one C call per kernel.

Each function takes torch tensors that live on the GPU, checks device, dtype,
contiguity and the sizes the kernel takes, and launches on torch's current
stream.  A size a kernel refuses raises ``KernelSizeError`` with the kernel's name
and the offending numbers; nothing here falls back to torch or to the CPU.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .build import BuildError, build_library

F32, BF16 = 0, 1
STATUS_BITS = {
    1: "a token id outside the embedding table",
    2: "a page id outside the pool where a live position needs one",
    4: "a negative position or sequence index, or a position beyond the block table's row",
    8: "a row of logits without a comparable value (all NaN)",
    16: "a bounded wait inside a kernel ran out (the kernel gave up cleanly)",
}


class KernelError(RuntimeError):
    pass


class KernelSizeError(KernelError):
    pass


_lib = None
_lib_path = None
_lock = threading.Lock()

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_c_ll, _c_ull = ctypes.c_longlong, ctypes.c_ulonglong

_SIGNATURES = {
    "q3_embed": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_add_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "q3_add_rmsnorm_rows": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                            _c_float, _c_void_p],
    "q3_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "q3_gemm_f32_nt": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_rope_table": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "q3_qkv_post": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                    _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                    _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "q3_attn_ref": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                    _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                    _c_void_p, _c_void_p],
    "q3_attn_decode": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                       _c_void_p, _c_void_p],
    "q3_attn_decode_tma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                           _c_void_p, _c_void_p],
    "q3_attn_decode_tma_qkv": [_c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                               _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_int, _c_float, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_attn_prefill": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p,
                        _c_void_p],
    "q3_attn_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "q3_swiglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_gemm_tc": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                   _c_void_p],
    "q3_gemm_tc_pair": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                        _c_void_p],
    "q3_gemm_tc_qkv": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                       _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                       _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_gemm_skinny": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_gemm_skinny_fused": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                             _c_int, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "q3_sample": [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ull, _c_int,
                  _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p],
}


_WAIT_TEST = ("q3_gemm_tc_wait_test", "q3_attn_tc_wait_test", "q3_attn_decode_tma_wait_test")


def library() -> ctypes.CDLL:
    """The loaded kernel library; compiles it at the first call if it is not built yet."""
    global _lib, _lib_path
    if _lib is None:
        with _lock:
            if _lib is None:
                try:
                    path = build_library()
                except BuildError as e:
                    raise KernelError(str(e)) from None
                lib = ctypes.CDLL(path)
                for name, argtypes in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.argtypes = argtypes
                    fn.restype = _c_int
                for name in _WAIT_TEST:
                    fn = getattr(lib, name)
                    fn.argtypes = [ctypes.c_uint, _c_int]
                    fn.restype = _c_int
                lib.q3_sm_count.argtypes = []
                lib.q3_sm_count.restype = _c_int
                lib.q3_attn_decode_blocks_per_sm.argtypes = [_c_int]
                lib.q3_attn_decode_blocks_per_sm.restype = _c_int
                lib.q3_sample_scratch_bytes.argtypes = [_c_int]
                lib.q3_sample_scratch_bytes.restype = _c_ll
                _lib, _lib_path = _Counting(lib), path
    return _lib


class _Counting:
    """The library with every launcher call counted (the benchmark reports launches per step)."""

    def __init__(self, lib):
        self._lib = lib
        self.calls = 0

    def __getattr__(self, name):
        if name not in _SIGNATURES:  # without declared argument types ctypes would cut pointers to 32 bits
            raise KernelError(f"{name}: no argument types declared for this entry point")
        fn = getattr(self._lib, name)

        def counted(*args):
            self.calls += 1
            return fn(*args)

        setattr(self, name, counted)
        return counted


def launch_count() -> int:
    """Kernel launches made through this module so far."""
    return library().calls


def library_path() -> Optional[str]:
    library()
    return _lib_path


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(name: str, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; the kernels run on the GPU only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")


def _done(kernel: str, code: int, detail: str = "") -> None:
    if code == 0:
        return
    if code == -2:
        raise KernelSizeError(f"{kernel}: size not taken by this kernel ({detail})")
    if code == -1:
        raise KernelError(f"{kernel}: dtype not taken ({detail})")
    if code == -3:
        raise KernelError(f"{kernel}: misaligned argument ({detail})")
    if code == -4:
        raise KernelSizeError(f"{kernel}: needs more scratch memory than is provided ({detail})")
    if code == -5:
        raise KernelError(f"{kernel}: the CUDA driver refused a tensor-map request ({detail})")
    raise KernelError(f"{kernel}: CUDA launch failed with error {code} ({detail})")


def set_wait_test(limit: int = 0, drop_copy: int = -1) -> None:
    """For tests of the path on which a kernel gives up a wait: every wait on an mbarrier in the TMA / tcgen05
    kernels polls ``limit`` times (0: the serving default of 2^24) and the loader of each leaves out its copy
    number ``drop_copy`` (-1: none), whose barrier then never completes.  Call it with no arguments to put the
    defaults back.  Synchronises the device."""
    torch.cuda.synchronize()
    for name in _WAIT_TEST:
        code = getattr(library()._lib, name)(int(limit), int(drop_copy))
        if code:
            raise KernelError(f"{name}: CUDA error {code}")
    torch.cuda.synchronize()


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "ok"


# ------------------------------------------------------------------ kernels
def embed(table: torch.Tensor, ids: torch.Tensor, resid: torch.Tensor, status: torch.Tensor) -> None:
    """resid[t] = float32(table[ids[t]])."""
    _check("embed.table", table)
    _check("embed.ids", ids, torch.int32)
    _check("embed.resid", resid, torch.float32)
    T, H = resid.shape
    V = table.shape[0]
    if table.shape[1] != H or ids.numel() != T:
        raise KernelError(f"embed: table {tuple(table.shape)}, ids {tuple(ids.shape)}, resid {tuple(resid.shape)}")
    code = library().q3_embed(table.data_ptr(), dtype_tag(table.dtype), ids.data_ptr(), resid.data_ptr(),
                              T, H, V, status.data_ptr(), _stream())
    _done("embed", code)


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float) -> None:
    """resid += delta (when given); out = rmsnorm(resid) * weight."""
    _check("add_rmsnorm.resid", resid, torch.float32)
    _check("add_rmsnorm.weight", weight, torch.float32)
    _check("add_rmsnorm.out", out)
    T, H = resid.shape
    if delta is not None:
        _check("add_rmsnorm.delta", delta, out.dtype)
        if tuple(delta.shape) != (T, H):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs stream {(T, H)}")
    if tuple(out.shape) != (T, H) or weight.numel() != H:
        raise KernelError(f"add_rmsnorm: out {tuple(out.shape)}, weight {tuple(weight.shape)}, stream {(T, H)}")
    code = library().q3_add_rmsnorm(resid.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(),
                                    dtype_tag(out.dtype), T, H, float(eps), _stream())
    _done("add_rmsnorm", code, f"width {H}")


def add_rmsnorm_rows(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                     rows: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out[r] = rmsnorm(resid[rows[r]] + delta[rows[r]]) * weight; resid is left as it is."""
    _check("add_rmsnorm_rows.resid", resid, torch.float32)
    _check("add_rmsnorm_rows.weight", weight, torch.float32)
    _check("add_rmsnorm_rows.rows", rows, torch.int32)
    _check("add_rmsnorm_rows.out", out)
    T, H = resid.shape
    R = rows.numel()
    if delta is not None:
        _check("add_rmsnorm_rows.delta", delta, out.dtype)
        if tuple(delta.shape) != (T, H):
            raise KernelError(f"add_rmsnorm_rows: delta {tuple(delta.shape)} vs stream {(T, H)}")
    if tuple(out.shape) != (R, H) or weight.numel() != H:
        raise KernelError(f"add_rmsnorm_rows: out {tuple(out.shape)}, rows {R}, width {H}")
    if R == 0:
        return
    code = library().q3_add_rmsnorm_rows(resid.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(),
                                         dtype_tag(out.dtype), rows.data_ptr(), R, H, float(eps), _stream())
    _done("add_rmsnorm_rows", code, f"width {H}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out[r] = rmsnorm(x[r]) * weight over the last dimension."""
    _check("rmsnorm.x", x)
    _check("rmsnorm.out", out, x.dtype)
    _check("rmsnorm.weight", weight, torch.float32)
    dim = x.shape[-1]
    rows = x.numel() // dim if dim else 0
    if out.shape != x.shape or weight.numel() != dim:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, out {tuple(out.shape)}, weight {tuple(weight.shape)}")
    code = library().q3_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_tag(x.dtype), rows, dim,
                                float(eps), _stream())
    _done("rmsnorm", code)


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in plain float32 (no tensor cores)."""
    _check("gemm_f32_nt.a", a, torch.float32)
    _check("gemm_f32_nt.w", w, torch.float32)
    _check("gemm_f32_nt.out", out, torch.float32)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_f32_nt: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = library().q3_gemm_f32_nt(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, K, K, N, _stream())
    _done("gemm_f32_nt", code, f"M {M} N {N} K {K}")


def qkv_post(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
             q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
             inv_freq: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
             tok_seq: torch.Tensor, block_table: torch.Tensor, num_q_heads: int, num_kv_heads: int,
             head_dim: int, write_kv: bool, status: torch.Tensor, cos_sin: Optional[torch.Tensor] = None) -> None:
    """Head norm, rotation, q to its buffer and k/v into their pages, in one pass over qkv.
    ``cos_sin``: the table of ``rope_table`` for the same positions and inv_freq (optional)."""
    _check("qkv_post.qkv", qkv)
    _check("qkv_post.q_out", q_out, qkv.dtype)
    _check("qkv_post.k_pages", k_pages, qkv.dtype)
    _check("qkv_post.v_pages", v_pages, qkv.dtype)
    _check("qkv_post.positions", positions, torch.int32)
    _check("qkv_post.tok_seq", tok_seq, torch.int32)
    _check("qkv_post.block_table", block_table, torch.int32)
    T = qkv.shape[0]
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or q_out.numel() != T * num_q_heads * head_dim:
        raise KernelError(f"qkv_post: qkv {tuple(qkv.shape)} expected [T, {width}]; q_out {tuple(q_out.shape)}")
    num_pages, hkv, page_size, d = k_pages.shape
    if hkv != num_kv_heads or d != head_dim or v_pages.shape != k_pages.shape:
        raise KernelError(f"qkv_post: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} "
                          f"vs heads {num_kv_heads} x {head_dim}")
    if positions.numel() != T or tok_seq.numel() != T or block_table.dim() != 2:
        raise KernelError("qkv_post: positions / tok_seq must have one entry per token; block_table is 2-D")
    for name, wt in (("q_weight", q_weight), ("k_weight", k_weight)):
        if wt is not None:
            _check(f"qkv_post.{name}", wt, torch.float32)
            if wt.numel() != head_dim:
                raise KernelError(f"qkv_post: {name} has {wt.numel()} elements, head_dim is {head_dim}")
    if inv_freq is not None:
        _check("qkv_post.inv_freq", inv_freq, torch.float32)
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError(f"qkv_post: inv_freq has {inv_freq.numel()} entries, rotary_dim is {rotary_dim}")
    if cos_sin is not None:
        _check("qkv_post.cos_sin", cos_sin, torch.float32)
        if inv_freq is None or tuple(cos_sin.shape) != (T, rotary_dim):
            raise KernelError(f"qkv_post: cos_sin {tuple(cos_sin.shape)} expected [{T}, {rotary_dim}] with inv_freq")
    code = library().q3_qkv_post(
        qkv.data_ptr(), dtype_tag(qkv.dtype), T, num_q_heads, num_kv_heads, head_dim, _ptr(q_weight),
        _ptr(k_weight), float(eps), _ptr(inv_freq), _ptr(cos_sin), int(rotary_dim), positions.data_ptr(), tok_seq.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, k_pages.data_ptr(), v_pages.data_ptr(),
        num_pages, q_out.data_ptr(), 1 if write_kv else 0, status.data_ptr(), _stream())
    _done("qkv_post", code, f"head_dim {head_dim}, rotary_dim {rotary_dim}")


def rope_table(inv_freq: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
    """table[t] = cos(positions[t] * inv_freq) then sin(...): float32 [T, 2 * len(inv_freq)]."""
    _check("rope_table.inv_freq", inv_freq, torch.float32)
    _check("rope_table.positions", positions, torch.int32)
    _check("rope_table.table", table, torch.float32)
    T, half = positions.numel(), inv_freq.numel()
    if tuple(table.shape) != (T, 2 * half):
        raise KernelError(f"rope_table: table {tuple(table.shape)} expected [{T}, {2 * half}]")
    code = library().q3_rope_table(inv_freq.data_ptr(), positions.data_ptr(), table.data_ptr(), T, half, _stream())
    _done("rope_table", code)


def attn_ref(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
             q_start: torch.Tensor, kv_len: torch.Tensor, tok_seq: torch.Tensor,
             block_table: torch.Tensor, scale: float, window: int, status: torch.Tensor) -> None:
    """Plain paged causal attention (one warp per query and head); any head_dim up to 512."""
    _check("attn_ref.q", q)
    _check("attn_ref.out", out, q.dtype)
    _check("attn_ref.k_pages", k_pages, q.dtype)
    _check("attn_ref.v_pages", v_pages, q.dtype)
    for name, t in (("q_start", q_start), ("kv_len", kv_len), ("tok_seq", tok_seq), ("block_table", block_table)):
        _check(f"attn_ref.{name}", t, torch.int32)
    T, Hq, D = q.shape
    num_pages, Hkv, page_size, d = k_pages.shape
    if d != D or v_pages.shape != k_pages.shape or out.numel() != q.numel():
        raise KernelError(f"attn_ref: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    code = library().q3_attn_ref(q.data_ptr(), dtype_tag(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
                                 out.data_ptr(), q_start.data_ptr(), kv_len.data_ptr(), tok_seq.data_ptr(),
                                 block_table.data_ptr(), block_table.shape[1], page_size, num_pages, T, Hq, Hkv,
                                 D, float(scale), int(window), status.data_ptr(), _stream())
    _done("attn_ref", code, f"heads {Hq}/{Hkv}, head_dim {D}")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave8: bool = False) -> None:
    """out = up * silu(gate); gate = first half of the columns and up = second half, or with
    ``interleave8`` alternating blocks of eight columns (gate, up, gate, up, ...)."""
    _check("swiglu.gate_up", gate_up)
    _check("swiglu.out", out, gate_up.dtype)
    T, two_i = gate_up.shape
    if two_i % 2 or tuple(out.shape) != (T, two_i // 2):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    code = library().q3_swiglu(gate_up.data_ptr(), out.data_ptr(), dtype_tag(out.dtype), T, two_i // 2,
                               1 if interleave8 else 0, _stream())
    _done("swiglu", code, f"width {two_i // 2}")


SKINNY_MAX_ROWS = 16  # rows of the few-rows product (two tiles of eight tokens)


def gemm_skinny_takes(rows: int, weight: torch.Tensor) -> bool:
    return rows <= SKINNY_MAX_ROWS and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu_blocks: bool = False) -> None:
    """out[T, N] = x[T, K] @ w[N, K]^T for T <= 16, bfloat16 in, out bfloat16 or float32.
    ``swiglu_blocks``: w's rows alternate gate/up in blocks of eight and out is [T, N / 2]."""
    _check("gemm_skinny.x", x, torch.bfloat16)
    _check("gemm_skinny.w", w, torch.bfloat16)
    _check("gemm_skinny.out", out)
    T, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if swiglu_blocks else N
    if w.shape[1] != K or tuple(out.shape) != (T, want_cols) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    code = library().q3_gemm_skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, want_cols,
                                    1 if out.dtype == torch.float32 else 0, 1 if swiglu_blocks else 0, _stream())
    _done("gemm_skinny", code, f"T {T} N {N} K {K}")


SUMSQ_ROWS = 16  # row pitch of the partial sums of squares that the fused few-rows products exchange


def sumsq_parts(features: int) -> int:
    """Partial sums per row that ``gemm_skinny_into_stream`` leaves for a stream ``features`` wide."""
    return (features + 15) // 16


def gemm_skinny_normed_pays(rows: int, weight: torch.Tensor) -> bool:
    """Whether a decode step without norm kernels is the faster one for this many rows and this reduction
    length: always with one token tile (up to 8 rows); with two only while the reduction is short, where the
    product with two token tiles is not yet short of registers (measured: profiles/decode_step_rules.md)."""
    return rows <= 8 or weight.shape[1] <= 3072


def gemm_skinny_normed(scaled: torch.Tensor, sumsq: torch.Tensor, parts: int, eps: float, w: torch.Tensor,
                       out: torch.Tensor, swiglu_blocks: bool = False) -> None:
    """out = rmsnorm(stream) @ w^T for up to 16 rows without a norm kernel.  ``scaled`` is the stream times
    the norm's weight in bfloat16 and ``sumsq[p, t]`` for ``p < parts`` are partial sums of squares of the
    stream's row ``t``, both as ``gemm_skinny_into_stream`` leaves them; the product of ``scaled`` is multiplied
    by the row's 1 / rms = 1 / sqrt(sum / K + eps) before it is stored.  ``swiglu_blocks`` as in ``gemm_skinny``."""
    _check("gemm_skinny_normed.scaled", scaled, torch.bfloat16)
    _check("gemm_skinny_normed.sumsq", sumsq, torch.float32)
    _check("gemm_skinny_normed.w", w, torch.bfloat16)
    _check("gemm_skinny_normed.out", out, torch.bfloat16)
    T, K = scaled.shape
    N = w.shape[0]
    want_cols = N // 2 if swiglu_blocks else N
    if (w.shape[1] != K or tuple(out.shape) != (T, want_cols) or sumsq.dim() != 2
            or sumsq.shape[1] != SUMSQ_ROWS or not 0 < parts <= sumsq.shape[0]):
        raise KernelError(f"gemm_skinny_normed: operand {tuple(scaled.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"sums {tuple(sumsq.shape)} of which {parts}")
    code = library().q3_gemm_skinny_fused(scaled.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, want_cols,
                                          4 if swiglu_blocks else 3, sumsq.data_ptr(), int(parts), float(eps), None, None,
                                          None, _stream())
    _done("gemm_skinny_normed", code, f"T {T} N {N} K {K}")


def gemm_skinny_into_stream(x: torch.Tensor, w: torch.Tensor, stream: torch.Tensor, sumsq: torch.Tensor,
                            next_weight: Optional[torch.Tensor] = None, scaled: Optional[torch.Tensor] = None) -> int:
    """stream += x @ w^T for up to 16 rows (x, w bfloat16; stream float32), and ``sumsq[p, t]`` = the sum of
    squares of the 16 new values ``stream[t, 16 p : 16 p + 16]``; returns the number of such parts.  With
    ``next_weight`` (the weight of the norm that comes next) and ``scaled`` (bfloat16, like stream):
    ``scaled = stream * next_weight``, rounded once: the operand of ``gemm_skinny_normed``."""
    _check("gemm_skinny_into_stream.x", x, torch.bfloat16)
    _check("gemm_skinny_into_stream.w", w, torch.bfloat16)
    _check("gemm_skinny_into_stream.stream", stream, torch.float32)
    _check("gemm_skinny_into_stream.sumsq", sumsq, torch.float32)
    T, K = x.shape
    N = w.shape[0]
    parts = sumsq_parts(N)
    if (w.shape[1] != K or tuple(stream.shape) != (T, N) or sumsq.dim() != 2 or sumsq.shape[1] != SUMSQ_ROWS
            or sumsq.shape[0] < parts or (next_weight is None) != (scaled is None)):
        raise KernelError(f"gemm_skinny_into_stream: x {tuple(x.shape)}, w {tuple(w.shape)}, stream "
                          f"{tuple(stream.shape)}, sums {tuple(sumsq.shape)}")
    if scaled is not None:
        _check("gemm_skinny_into_stream.next_weight", next_weight, torch.float32)
        _check("gemm_skinny_into_stream.scaled", scaled, torch.bfloat16)
        if next_weight.numel() != N or tuple(scaled.shape) != (T, N):
            raise KernelError(f"gemm_skinny_into_stream: next weight {tuple(next_weight.shape)}, scaled "
                              f"{tuple(scaled.shape)} for a stream {(T, N)}")
    code = library().q3_gemm_skinny_fused(x.data_ptr(), w.data_ptr(), stream.data_ptr(), T, N, K, N, 2, None, 0,
                                          0.0, sumsq.data_ptr(), _ptr(next_weight), _ptr(scaled), _stream())
    _done("gemm_skinny_into_stream", code, f"T {T} N {N} K {K}")
    return parts


def sample(logits: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
           temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           request_key: Optional[torch.Tensor] = None, position: Optional[torch.Tensor] = None,
           seed: int = 0) -> None:
    """One token per row of float32 logits: argmax where temperature <= 0, else a Gumbel-max draw
    (among the top_k largest logits where top_k > 0)."""
    _check("sample.logits", logits, torch.float32)
    _check("sample.out", out, torch.int32)
    R, V = logits.shape
    if out.numel() != R:
        raise KernelError(f"sample: {R} rows of logits, {out.numel()} outputs")
    if temperature is not None:
        _check("sample.temperature", temperature, torch.float32)
        if request_key is None or position is None:
            raise KernelError("sample: a temperature needs request_key and position")
        _check("sample.request_key", request_key, torch.int64)
        _check("sample.position", position, torch.int32)
    if top_k is not None:
        _check("sample.top_k", top_k, torch.int32)
    scratch = _sample_scratch(logits.device, R)
    code = library().q3_sample(logits.data_ptr(), R, V, V, _ptr(temperature), _ptr(top_k), _ptr(request_key),
                               _ptr(position), int(seed) & 0xFFFFFFFFFFFFFFFF,
                               1 if (top_k is not None and temperature is not None) else 0, scratch.data_ptr(),
                               scratch.numel(), out.data_ptr(), status.data_ptr(), _stream())
    _done("sample", code)


_SAMPLE_SCRATCH = {}


def _sample_scratch(device: torch.device, rows: int) -> torch.Tensor:
    """Zero-filled working memory of the sampling kernels for up to ``rows`` rows (they leave it zeroed)."""
    have = _SAMPLE_SCRATCH.get(device)
    need = int(library()._lib.q3_sample_scratch_bytes(max(rows, 8)))
    if have is None or have.numel() < need:
        have = torch.zeros(need, dtype=torch.uint8, device=device)
        _SAMPLE_SCRATCH[device] = have
    return have


def rope(x: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, positions: torch.Tensor,
         out: torch.Tensor, status: torch.Tensor) -> None:
    """out = rotate-half rotary encoding of x[T, heads, D] at `positions` (no norm, no cache)."""
    _check("rope.x", x)
    _check("rope.out", out, x.dtype)
    _check("rope.inv_freq", inv_freq, torch.float32)
    _check("rope.positions", positions, torch.int32)
    T, heads, d = x.shape
    if out.shape != x.shape or positions.numel() != T or inv_freq.numel() * 2 != rotary_dim:
        raise KernelError(f"rope: x {tuple(x.shape)}, out {tuple(out.shape)}, positions {positions.numel()}, "
                          f"inv_freq {inv_freq.numel()}, rotary_dim {rotary_dim}")
    code = library().q3_qkv_post(
        x.data_ptr(), dtype_tag(x.dtype), T, heads, 0, d, None, None, 0.0, inv_freq.data_ptr(), None, int(rotary_dim),
        positions.data_ptr(), positions.data_ptr(), None, 1, 1, None, None, 0, out.data_ptr(), 0,
        status.data_ptr(), _stream())
    _done("rope", code, f"head_dim {d}, rotary_dim {rotary_dim}")


def gemm_tc_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0


def gemm_tc_swiglu_pays(rows: int, weight: torch.Tensor) -> Optional[str]:
    """Which of the engine's tcgen05 gate/up products with SwiGLU in the epilogue is the faster way for a
    prompt portion: "pair" (pairs of CTAs on 256 x 256 tiles), "single" (one CTA on 128 x 256) or None (the
    library's product followed by the gate kernel).  The fused forms save the gate kernel's pass over the
    [rows, 2 I] product.  The pair form runs at the library's rate and wins from 1,024 rows at every width and
    from 512 where the reduction is long; the single-CTA form falls behind the library when the reduction is
    long or the rows are many, and is kept for the short portions of a narrow model
    (measured: profiles/gemm_tc_swiglu__prefill_2048.md)."""
    narrow = weight.shape[1] <= 1536
    if rows >= 1024 or (rows >= 512 and not narrow):
        return "pair"
    return "single" if narrow and rows >= 128 else None


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
            swiglu_blocks: bool = False, pair: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in TMEM).
    ``swiglu_blocks``: w's rows alternate gate/up in blocks of eight and out is [M, N / 2].
    ``pair``: by pairs of CTAs on 256 x 256 tiles (the paired instruction) instead of single CTAs."""
    _check("gemm_tc.x", x, torch.bfloat16)
    _check("gemm_tc.w", w, torch.bfloat16)
    _check("gemm_tc.out", out)
    M, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if swiglu_blocks else N
    if w.shape[1] != K or tuple(out.shape) != (M, want_cols) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    entry = library().q3_gemm_tc_pair if pair else library().q3_gemm_tc
    code = entry(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, want_cols,
                 1 if out.dtype == torch.float32 else 0, 1 if swiglu_blocks else 0, status.data_ptr(), _stream())
    _done("gemm_tc", code, f"M {M} N {N} K {K}{' pair' if pair else ''}")


# ------------------------------------------------------------------ fast bfloat16 attention
MAX_DECODE_SPLITS = 32


def gemm_tc_qkv_takes(rows: int, x: torch.Tensor, weight: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether the QKV projection with head norm, rotation and cache write in its epilogue takes this
    case: a prompt portion (128 rows or more) in bfloat16, heads of 64 or 128, rotated whole or not at all."""
    return (rows >= 128 and gemm_tc_takes(x, weight) and head_dim in (64, 128) and rotary_dim in (0, head_dim))


def gemm_tc_qkv_pays(rows: int, weight: torch.Tensor) -> Optional[str]:
    """Which projection with ``qkv_post`` as its epilogue is the faster way for a prompt portion: "pair"
    (pairs of CTAs on tiles of 256 rows), "single" (one CTA per tile) or None (the library's product, then
    ``qkv_post``).  The fused forms save ``qkv_post``'s pass over the projection and a launch.  Inside the
    step they win from 256 rows at a reduction up to 1,536 (3 to 6 % of the step); where the reduction is
    longer the step showed no gain over the library's product beyond its spread from run to run
    (profiles/gemm_tc_qkv__prefill_2048.md, profiles/gemm_tc_pair__products.md)."""
    if weight.shape[1] > 1536 or rows < 256:
        return None
    return "pair" if rows >= 1024 else "single"


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                cos_sin: Optional[torch.Tensor], positions: torch.Tensor, tok_seq: torch.Tensor,
                block_table: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool,
                status: torch.Tensor, pair: bool = False) -> None:
    """x[T, K] @ w[(Hq + 2 Hkv) D, K]^T on the tensor cores with ``qkv_post`` as the epilogue: the
    projection is rounded to bfloat16, normed and rotated head by head and written to ``q_out`` and the
    cache pages; it is never stored itself (``gemm_tc_qkv_pays`` says where the attention part takes it).
    ``pair``: by pairs of CTAs on tiles of 256 rows (the paired instruction) instead of single CTAs."""
    for name, t in (("x", x), ("w", w), ("q_out", q_out), ("k_pages", k_pages), ("v_pages", v_pages)):
        _check(f"gemm_tc_qkv.{name}", t, torch.bfloat16)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("block_table", block_table)):
        _check(f"gemm_tc_qkv.{name}", t, torch.int32)
    T, K = x.shape
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    num_pages, hkv, page_size, d = k_pages.shape
    if (tuple(w.shape) != (width, K) or q_out.numel() != T * num_q_heads * head_dim or hkv != num_kv_heads
            or d != head_dim or v_pages.shape != k_pages.shape or positions.numel() != T or tok_seq.numel() != T
            or block_table.dim() != 2):
        raise KernelError(f"gemm_tc_qkv: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}, "
                          f"pages {tuple(k_pages.shape)}, heads {num_q_heads}/{num_kv_heads} x {head_dim}")
    for name, wt in (("q_weight", q_weight), ("k_weight", k_weight)):
        if wt is not None:
            _check(f"gemm_tc_qkv.{name}", wt, torch.float32)
            if wt.numel() != head_dim:
                raise KernelError(f"gemm_tc_qkv: {name} has {wt.numel()} elements, head_dim is {head_dim}")
    if cos_sin is not None:
        _check("gemm_tc_qkv.cos_sin", cos_sin, torch.float32)
        if tuple(cos_sin.shape) != (T, head_dim):
            raise KernelError(f"gemm_tc_qkv: cos_sin {tuple(cos_sin.shape)} expected [{T}, {head_dim}]")
    code = library().q3_gemm_tc_qkv(
        x.data_ptr(), w.data_ptr(), T, K, num_q_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight),
        float(eps), _ptr(cos_sin), positions.data_ptr(), tok_seq.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, k_pages.data_ptr(), v_pages.data_ptr(), num_pages, q_out.data_ptr(),
        1 if write_kv else 0, 1 if pair else 0, status.data_ptr(), _stream())
    _done("gemm_tc_qkv", code, f"T {T} K {K} heads {num_q_heads}/{num_kv_heads} x {head_dim}{' pair' if pair else ''}")


def fast_attention_takes(dtype: torch.dtype, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core kernels take this shape (else the plain kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and num_q_heads % num_kv_heads == 0 and num_q_heads // num_kv_heads <= 16)


_DEVICE_FACTS = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once)."""
    key = ("sms", torch.cuda.current_device())
    if key not in _DEVICE_FACTS:
        _DEVICE_FACTS[key] = max(1, int(library()._lib.q3_sm_count()))
    return _DEVICE_FACTS[key]


def decode_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the cp.async decode kernel that one SM holds at once, as the CUDA runtime reckons it from the
    compiled kernel (registers, shared memory); asked once per head size."""
    key = ("decode blocks", torch.cuda.current_device(), head_dim)
    if key not in _DEVICE_FACTS:
        _DEVICE_FACTS[key] = max(1, int(library()._lib.q3_attn_decode_blocks_per_sm(int(head_dim))))
    return _DEVICE_FACTS[key]


def decode_tma_takes(head_dim: int, page_size: int) -> bool:
    """Whether the decode kernel with the TMA loader takes this shape (else the cp.async one runs)."""
    return head_dim in (64, 128) and page_size % 16 == 0


def decode_takes_raw_qkv(dtype: torch.dtype, num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         num_tokens: int, num_seqs: int, num_decode: int) -> bool:
    """Whether the decode attention kernel can do the work of ``qkv_post`` itself: every row of the step
    brings one token and the kernel with the TMA loader takes the shape."""
    return (num_tokens == num_seqs == num_decode and num_decode > 0
            and fast_attention_takes(dtype, num_q_heads, num_kv_heads, head_dim)
            and decode_tma_takes(head_dim, page_size))


DECODE_SATURATING = 2.3    # blocks per SM that together take tiles as fast as the memory gives them
DECODE_LATER_WAVE = 5      # what every wave of blocks after the first costs beside its tiles, in tiles
DECODE_WIDE_GRID = 20      # what the form of the kernel for more blocks per SM costs beside its tiles
DECODE_LONG_BLOCK = (0.15, 128)  # a single wave of that form: per tile of a block beyond so many


def decode_splits(num_seqs: int, num_kv_heads: int, max_kv_len: int, window: int, head_dim: int = 128,
                  blocks_per_sm: Optional[int] = None, wide_blocks_per_sm: Optional[int] = None) -> int:
    """How many ranges a sequence's keys are cut into.  Blocks run in waves of (SMs x blocks per SM).  A
    block alone walks its 16-key tiles at its own pace; ``DECODE_SATURATING`` blocks per SM together take
    tiles as fast as the memory gives them, and more blocks then only share that rate; every wave after the
    first costs a start.  So a wave of n blocks of L tiles costs max(L, n L / saturating), and the count with
    the least sum over its waves wins, the smaller count on a tie.  ``wide_blocks_per_sm``: the kernel has a
    form with that many (smaller) blocks per SM, which the launcher takes for a grid that ``blocks_per_sm``
    do not hold at once.  The constants are fitted to sweeps of the decode step over batch and context
    (profiles/attn_decode_tma__decode_b8_ctx4096.md)."""
    span = min(max_kv_len, window) if window and window > 0 else max_kv_len
    tiles = max(1, -(-span // 16))
    sms = sm_count()
    narrow = sms * (blocks_per_sm or decode_blocks_per_sm(head_dim))
    saturating = DECODE_SATURATING * sms
    pairs = max(1, num_seqs * num_kv_heads)
    best, best_cost = 1, None
    for s in range(1, MAX_DECODE_SPLITS + 1):
        if s > 1 and tiles // s < 4:
            break
        per_block = -(-tiles // s)
        blocks = pairs * s
        wide = wide_blocks_per_sm is not None and blocks > narrow
        slots = sms * wide_blocks_per_sm if wide else narrow
        full, rest = divmod(blocks, slots)
        waves = full + (1 if rest else 0)
        cost = full * max(per_block, slots * per_block / saturating) + DECODE_LATER_WAVE * (waves - 1)
        if rest:
            cost += max(per_block, rest * per_block / saturating)
        if wide:
            cost += DECODE_WIDE_GRID
            if waves == 1:
                cost += DECODE_LONG_BLOCK[0] * max(0, per_block - DECODE_LONG_BLOCK[1])
        if best_cost is None or cost < best_cost - 1e-6:
            best, best_cost = s, cost
    return best


def decode_partial_numel(num_seqs: int, num_q_heads: int, head_dim: int) -> int:
    return num_seqs * num_q_heads * MAX_DECODE_SPLITS * (head_dim + 2)


def _attn_common(name, q, k_pages, v_pages, out, q_start, kv_len, block_table):
    _check(f"{name}.q", q, torch.bfloat16)
    _check(f"{name}.out", out, torch.bfloat16)
    _check(f"{name}.k_pages", k_pages, torch.bfloat16)
    _check(f"{name}.v_pages", v_pages, torch.bfloat16)
    for nm, t in (("q_start", q_start), ("kv_len", kv_len), ("block_table", block_table)):
        _check(f"{name}.{nm}", t, torch.int32)
    T, Hq, D = q.shape
    num_pages, Hkv, page_size, d = k_pages.shape
    if d != D or v_pages.shape != k_pages.shape or out.numel() != q.numel() or block_table.dim() != 2:
        raise KernelError(f"{name}: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    return T, Hq, D, num_pages, Hkv, page_size


def attn_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                partial: Optional[torch.Tensor], q_start: torch.Tensor, kv_len: torch.Tensor,
                block_table: torch.Tensor, num_seqs: int, scale: float, window: int, num_splits: int,
                status: torch.Tensor, loader: str = "cp_async", raw_qkv=None) -> None:
    """Split-KV tensor-core attention for the first ``num_seqs`` rows, one query token each.
    ``raw_qkv = (qkv, q_weight, k_weight, eps, cos_sin, write_kv)`` (TMA loader only): ``q`` only gives the
    shape; the kernel norms and rotates the query from the raw projection ``qkv[T, (Hq + 2 Hkv) D]`` itself
    and makes, stores and uses the new key and value (the work of ``qkv_post`` for these tokens).
    ``loader``: ``"cp_async"`` (every warp copies its own tiles) or ``"tma"`` (a loader warp feeds a
    ring of stages through TMA; head size 64 / 128 and pages that are multiples of 16 only)."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_decode", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if num_seqs > kv_len.numel() or num_seqs > block_table.shape[0]:
        raise KernelError(f"attn_decode: {num_seqs} sequences, {kv_len.numel()} lengths")
    if num_splits > 1:
        if partial is None:
            raise KernelError("attn_decode: more than one split needs scratch memory")
        _check("attn_decode.partial", partial, torch.float32)
        if partial.numel() < num_seqs * Hq * num_splits * (D + 2):
            raise KernelError(f"attn_decode: scratch of {partial.numel()} floats is too small for {num_seqs} "
                              f"sequences x {Hq} heads x {num_splits} splits")
    if raw_qkv is not None:
        qkv, q_weight, k_weight, eps, cos_sin, write_kv = raw_qkv
        if loader != "tma":
            raise KernelError("attn_decode: only the kernel with the TMA loader takes the raw projection")
        _check("attn_decode.qkv", qkv, torch.bfloat16)
        if tuple(qkv.shape) != (T, (Hq + 2 * Hkv) * D) or num_seqs > T:
            raise KernelError(f"attn_decode: raw projection {tuple(qkv.shape)} for {T} tokens of {Hq}+2x{Hkv} heads of {D}")
        for nm, t, n in (("q_weight", q_weight, D), ("k_weight", k_weight, D), ("cos_sin", cos_sin, T * D)):
            if t is not None:
                _check(f"attn_decode.{nm}", t, torch.float32)
                if t.numel() != n:
                    raise KernelError(f"attn_decode: {nm} has {t.numel()} values, {n} expected")
        code = library().q3_attn_decode_tma_qkv(
            qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos_sin), 1 if write_kv else 0,
            k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), _ptr(partial), q_start.data_ptr(), kv_len.data_ptr(),
            block_table.data_ptr(), block_table.shape[1], page_size, num_pages, num_seqs, Hq, Hkv, D, float(scale),
            int(window), int(num_splits), status.data_ptr(), _stream())
        _done("attn_decode", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}, raw projection")
        return
    fn = library().q3_attn_decode_tma if loader == "tma" else library().q3_attn_decode
    code = fn(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
              _ptr(partial), q_start.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], page_size, num_pages, num_seqs, Hq, Hkv, D, float(scale),
              int(window), int(num_splits), status.data_ptr(), _stream())
    _done("attn_decode", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}, loader {loader}")


def attn_prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                 q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, num_seqs: int,
                 max_q_len: int, scale: float, window: int, status: torch.Tensor) -> None:
    """Tensor-core attention for ``num_seqs`` rows of any query length (q_start has num_seqs + 1 entries)."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_prefill", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if q_start.numel() < num_seqs + 1 or kv_len.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError(f"attn_prefill: {num_seqs} sequences, q_start {q_start.numel()}, kv_len {kv_len.numel()}")
    code = library().q3_attn_prefill(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                     q_start.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
                                     block_table.shape[1], page_size, num_pages, num_seqs, int(max_q_len), Hq, Hkv, D,
                                     float(scale), int(window), status.data_ptr(), _stream())
    _done("attn_prefill", code, f"heads {Hq}/{Hkv}, head_dim {D}")


def attn_tc_takes(head_dim: int, page_size: int, window: int) -> bool:
    """Whether the tcgen05 portion kernel takes this shape (else the mma.sync one runs)."""
    return head_dim in (64, 128) and page_size in (8, 16, 32, 64) and not (window and window > 0)


def attn_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
            q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, num_seqs: int,
            max_q_len: int, scale: float, status: torch.Tensor) -> None:
    """Portion attention on the tcgen05 tensor cores: TMA-fed pages, S and O in tensor memory."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_tc", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if q_start.numel() < num_seqs + 1 or kv_len.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError(f"attn_tc: {num_seqs} sequences, q_start {q_start.numel()}, kv_len {kv_len.numel()}")
    code = library().q3_attn_tc(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                q_start.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                page_size, num_pages, num_seqs, int(max_q_len), Hq, Hkv, D, float(scale),
                                status.data_ptr(), _stream())
    _done("attn_tc", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}")


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                    q_start: torch.Tensor, kv_len: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                    num_seqs: int, num_decode: int, max_q_len: int, max_kv_len: int, scale: float, window: int,
                    status: torch.Tensor, partial: Optional[torch.Tensor] = None,
                    portion_kernel: str = "auto", decode_kernel: str = "auto", raw_qkv=None) -> None:
    """``raw_qkv``: see ``attn_decode``; only where ``decode_takes_raw_qkv`` says so.
    Causal attention of a mixed batch over the pages: rows [0, num_decode) bring one token each and
    go to the split-KV decode kernel, the rest to a portion kernel (tcgen05 where it takes the shape,
    else mma.sync; ``portion_kernel="mma"`` forces the latter); shapes no tensor-core kernel takes
    (and float32) go to the plain kernel."""
    T, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    if block_table.dim() != 2 or max_kv_len > block_table.shape[1] * k_pages.shape[2]:
        raise KernelError(f"paged_attention: the longest request has {max_kv_len} tokens, a block table row of "
                          f"{block_table.shape[-1]} pages of {k_pages.shape[2]} holds fewer")
    if not fast_attention_takes(q.dtype, Hq, Hkv, D):
        attn_ref(q, k_pages, v_pages, out, q_start, kv_len, tok_seq, block_table, scale, window, status)
        return
    if num_decode > 0:
        tma = decode_kernel != "cp_async" and decode_tma_takes(D, k_pages.shape[2])
        if tma:
            # The kernel is compiled for two, three and four blocks per SM (the last with fewer warps and
            # stages per block) and takes the smallest form that holds the grid at once, the last for all larger grids.
            splits = decode_splits(num_decode, Hkv, max_kv_len, window, D, blocks_per_sm=3, wide_blocks_per_sm=4)
        else:
            splits = decode_splits(num_decode, Hkv, max_kv_len, window, D)
        if partial is None or partial.numel() < num_decode * Hq * splits * (D + 2):
            splits = 1 if partial is None else max(1, partial.numel() // (num_decode * Hq * (D + 2)))
        attn_decode(q, k_pages, v_pages, out, partial, q_start, kv_len, block_table, num_decode, scale, window,
                    splits, status, loader="tma" if tma else "cp_async", raw_qkv=raw_qkv)
    elif raw_qkv is not None:
        raise KernelError("paged_attention: the raw projection is only taken by a step of single tokens")
    if num_seqs > num_decode:
        rest = (q_start[num_decode:], kv_len[num_decode:], block_table[num_decode:], num_seqs - num_decode, max_q_len)
        if portion_kernel != "mma" and attn_tc_takes(D, k_pages.shape[2], window):
            attn_tc(q, k_pages, v_pages, out, *rest, scale, status)
        else:
            attn_prefill(q, k_pages, v_pages, out, *rest, scale, window, status)
