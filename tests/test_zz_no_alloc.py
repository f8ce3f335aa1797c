"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory at the moment they need attention (all
memory already given to the cache pool, a fixed memory budget inside another program, a step with
a deadline): for them `q3_attn_decode_noalloc` keeps the split-KV scratch in an array inside the
library.  This test calls it twice in a row, with different shapes, and wants bit for bit what the
ordinary entry point (which takes the scratch from the caller) produces, and what a plain float64
restatement of attention gives within the bfloat16 tolerance of the kernel tests.  The free device
memory that the driver reports is read around every call (after one warm-up call, so that the
lazy loading of the kernels is not counted): it must not move.  It is named to be collected last;
it must pass alone in a fresh process as well as after every other test."""

import ctypes

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def _plain_attention(c, window):
    """The decode step restated: for every sequence the whole-sequence attention of the plain implementation
    over its cached keys and values in float64, of which the last row is the step's."""
    page = c["page_size"]
    rows = []
    for b, n in enumerate(c["kv_len"].tolist()):
        table = c["table"][b].tolist()
        k = torch.stack([c["k"][table[p // page], :, p % page] for p in range(n)]).double().cpu()
        v = torch.stack([c["v"][table[p // page], :, p % page] for p in range(n)]).double().cpu()
        q = torch.zeros(n, c["hq"], c["d"], dtype=torch.float64)
        q[-1] = c["q"][b].double().cpu()
        rows.append(plain.causal_attention(q, k, v, window or None)[-1])
    return torch.stack(rows)


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
    warm = cases[0][0]  # one call first: the driver loads the kernels' code at their first launch
    fn(warm["q"].data_ptr(), warm["k"].data_ptr(), warm["v"].data_ptr(), torch.empty_like(warm["q"]).data_ptr(),
       warm["q_start"].data_ptr(), warm["kv_len"].data_ptr(), warm["table"].data_ptr(), warm["table"].shape[1],
       warm["page_size"], warm["num_pages"], warm["q"].shape[0], warm["hq"], warm["hkv"], warm["d"], 1.0, 0, 2,
       status.data_ptr(), stream)
    torch.cuda.synchronize()
    for c, splits, window in cases:
        scale = c["d"] ** -0.5
        want = torch.empty_like(c["q"])
        partial = torch.empty(ops.decode_partial_numel(c["q"].shape[0], c["hq"], c["d"]), device="cuda")
        ops.attn_decode(c["q"], c["k"], c["v"], want, partial, c["q_start"], c["kv_len"], c["table"],
                        c["q"].shape[0], scale, window, splits, status)
        got = torch.full_like(c["q"], float("nan"))
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        code = fn(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), got.data_ptr(), c["q_start"].data_ptr(),
                  c["kv_len"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], c["page_size"], c["num_pages"],
                  c["q"].shape[0], c["hq"], c["hkv"], c["d"], scale, window, splits, status.data_ptr(), stream)
        assert code == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before, "the driver's free memory moved: something allocated"
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)  # the same kernels on the same inputs, only the scratch lies elsewhere
        exact = _plain_attention(c, window)
        err = float((got.double().cpu() - exact).abs().max()) / float(exact.abs().max())
        assert err <= 4e-3  # bfloat16 probabilities and output, as in the kernel tests
    assert int(status.item()) == 0
    # a call beyond the fixed scratch is refused and launches nothing
    c = cases[0][0]
    too_many = capacity // (c["q"].shape[0] * c["hq"] * (c["d"] + 2)) + 1
    code = fn(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), got.data_ptr(), c["q_start"].data_ptr(),
              c["kv_len"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], c["page_size"], c["num_pages"],
              c["q"].shape[0], c["hq"], c["hkv"], c["d"], 1.0, 0, int(too_many), status.data_ptr(), stream)
    assert code == -4
