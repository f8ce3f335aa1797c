"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory at the moment they need attention (all
memory already given to the cache pool, a fixed memory budget inside another program, a step with
a deadline): for them `q3_attn_decode_noalloc` keeps the split-KV scratch in an array inside the
library.  This test calls it twice in a row, with different shapes, and wants exactly what the
ordinary entry point (which takes the scratch from the caller) produces.  It is named to be
collected last; it must pass alone in a fresh process as well as after every other test."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, num_seqs, hq, hkv, d, page_size, lengths):
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_per_seq) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    tables, at = [], 0
    for n in pages_per_seq:
        tables.append(perm[at:at + n])
        at += n
    stride = max(pages_per_seq)
    table = torch.tensor([t + [-1] * (stride - len(t)) for t in tables], dtype=torch.int32)
    dev = "cuda"
    return dict(
        q=torch.randn(num_seqs, hq, d, generator=g).to(torch.bfloat16).to(dev),
        k=torch.randn(num_pages, hkv, page_size, d, generator=g).to(torch.bfloat16).to(dev),
        v=torch.randn(num_pages, hkv, page_size, d, generator=g).to(torch.bfloat16).to(dev),
        q_start=torch.arange(num_seqs + 1, dtype=torch.int32, device=dev),
        kv_len=torch.tensor(lengths, dtype=torch.int32, device=dev),
        table=table.to(dev), num_pages=num_pages, page_size=page_size, hq=hq, hkv=hkv, d=d)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from qwen3_from_scratch_b200.kernels import ops

    lib = ctypes.CDLL(ops.library_path())
    fn = lib.q3_attn_decode_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ctypes.c_float, ci, ci, vp, vp]
    fn.restype = ci
    lib.q3_attn_decode_noalloc_capacity.restype = ctypes.c_longlong
    capacity = lib.q3_attn_decode_noalloc_capacity()
    assert capacity == 4 << 20

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(_case(1, 5, 8, 2, 64, 16, [700, 33, 160, 1, 512]), 7, 0),
             (_case(2, 3, 16, 8, 128, 16, [1000, 999, 17]), 4, 300)]
    for c, splits, window in cases:
        scale = c["d"] ** -0.5
        want = torch.empty_like(c["q"])
        partial = torch.empty(ops.decode_partial_numel(c["q"].shape[0], c["hq"], c["d"]), device="cuda")
        ops.attn_decode(c["q"], c["k"], c["v"], want, partial, c["q_start"], c["kv_len"], c["table"],
                        c["q"].shape[0], scale, window, splits, status)
        got = torch.full_like(c["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        code = fn(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), got.data_ptr(), c["q_start"].data_ptr(),
                  c["kv_len"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], c["page_size"], c["num_pages"],
                  c["q"].shape[0], c["hq"], c["hkv"], c["d"], scale, window, splits, status.data_ptr(), stream)
        assert code == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        # the same kernels on the same inputs: the engine's bfloat16 tolerance is far more than needed
        err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
        assert err <= 4e-3
    assert int(status.item()) == 0
    # a call beyond the fixed scratch is refused and launches nothing
    c = cases[0][0]
    too_many = capacity // (c["q"].shape[0] * c["hq"] * (c["d"] + 2)) + 1
    code = fn(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), got.data_ptr(), c["q_start"].data_ptr(),
              c["kv_len"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], c["page_size"], c["num_pages"],
              c["q"].shape[0], c["hq"], c["hkv"], c["d"], 1.0, 0, int(too_many), status.data_ptr(), stream)
    assert code == -4
