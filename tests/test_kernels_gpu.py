"""Each kernel alone against a plain float32/float64 torch restatement of the same formula, at
sizes other than the engine's tiny models use (odd widths, head sizes in steps of 16, scattered
pages, ragged lengths)."""

import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative to the largest |expected| value: float32 kernels differ from float64 by summation
# order only; bfloat16 outputs are rounded once to 8 significant bits (2^-9 = 0.002) and, where
# inputs are bfloat16 too, the expectation is computed from the same rounded inputs.
TOL = {"float32": 2e-6, "bfloat16": 4e-3}


def ops():
    from qwen3_from_scratch_b200.kernels import ops as o
    return o


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype else t.to("cuda")


def close(got, want, dtype, scale=None, tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    scale = scale or max(float(want.abs().max()), 1e-9)
    err = float((got - want).abs().max()) / scale
    tol = tol if tol is not None else TOL[dtype]
    assert math.isfinite(err) and err <= tol, f"relative error {err:.3g} > {tol:g}"


def f32_accumulation_tol(k):
    """A float32 accumulator rounds once per step (2^-24 relative): over k steps the error walks to
    about sqrt(k) * 2^-24 of the sum's scale; twice that is the bound for products with float32 output."""
    return max(2e-6, 2 * math.sqrt(k) * 2.0 ** -24)


def status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", list(DT))
def test_embed(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 96, generator=g).to(DT[dtype])
    ids = torch.randint(0, 1000, (37,), generator=g, dtype=torch.int32)
    out = torch.empty(37, 96, device="cuda")
    st = status()
    ops().embed(dev(table), dev(ids), out, st)
    assert torch.equal(out.cpu(), table.float()[ids.long()])
    assert int(st.item()) == 0
    bad = ids.clone()
    bad[5] = 1000
    ops().embed(dev(table), dev(bad), out, st)
    assert int(st.item()) == 1 and float(out[5].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("width", [100, 2560, 6])
def test_add_rmsnorm(dtype, width):
    g = torch.Generator().manual_seed(1)
    T, eps = 37, 1e-5
    stream = torch.randn(T, width, generator=g) * 3
    delta = (torch.randn(T, width, generator=g)).to(DT[dtype])
    w = 1 + 0.1 * torch.randn(width, generator=g)
    s = dev(stream.clone())
    out = torch.empty(T, width, device="cuda", dtype=DT[dtype])
    ops().add_rmsnorm(s, dev(delta), dev(w), out, eps)
    total = stream.double() + delta.double()
    close(s, total, "float32")
    close(out, plain.rms_norm(total, w.double(), eps), dtype)
    # without a delta the stream is left alone
    s2 = dev(stream.clone())
    ops().add_rmsnorm(s2, None, dev(w), out, eps)
    assert torch.equal(s2.cpu(), stream)
    close(out, plain.rms_norm(stream.double(), w.double(), eps), dtype)
    # chosen rows, stream unchanged
    rows = torch.tensor([36, 0, 17, 17], dtype=torch.int32)
    s3 = dev(stream.clone())
    out_rows = torch.empty(4, width, device="cuda", dtype=DT[dtype])
    ops().add_rmsnorm_rows(s3, dev(delta), dev(w), dev(rows), out_rows, eps)
    assert torch.equal(s3.cpu(), stream)
    close(out_rows, plain.rms_norm(total[rows.long()], w.double(), eps), dtype)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("width", [128, 640, 1024, 2048, 2176])
def test_add_rmsnorm_many_rows(dtype, width):
    """Enough rows for the one-warp-per-row kernel (bfloat16, widths that are multiples of 128 up to
    2048); the other widths and float32 take the one-block-per-row kernel."""
    g = torch.Generator().manual_seed(11)
    T, eps = 200, 1e-6
    stream = torch.randn(T, width, generator=g) * 2
    delta = torch.randn(T, width, generator=g).to(DT[dtype])
    w = 1 + 0.1 * torch.randn(width, generator=g)
    s = dev(stream.clone())
    out = torch.empty(T, width, device="cuda", dtype=DT[dtype])
    ops().add_rmsnorm(s, dev(delta), dev(w), out, eps)
    total = stream.double() + delta.double()
    close(s, total, "float32")
    close(out, plain.rms_norm(total, w.double(), eps), dtype)
    rows = torch.randperm(T, generator=g)[:100].to(torch.int32)
    s3 = dev(stream.clone())
    out_rows = torch.empty(100, width, device="cuda", dtype=DT[dtype])
    ops().add_rmsnorm_rows(s3, dev(delta), dev(w), dev(rows), out_rows, eps)
    assert torch.equal(s3.cpu(), stream)
    close(out_rows, plain.rms_norm(total[rows.long()], w.double(), eps), dtype)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("rows", [24, 6000])
def test_add_rmsnorm_right_after_a_writer_of_the_stream(dtype, rows):
    """A norm reads the stream ahead of its wait on the launch before it unless that launch wrote the
    stream.  Three norms in a row (each writes what the next reads), and norms with one short launch
    of another kind between them (the writer is two launches back: long, so that it would still be
    running if the later norm could start before it ended)."""
    g = torch.Generator().manual_seed(12)
    width, eps = 1024, 1e-6
    stream = torch.randn(rows, width, generator=g)
    deltas = [torch.randn(rows, width, generator=g).to(DT[dtype]) for _ in range(3)]
    w = 1 + 0.1 * torch.randn(width, generator=g)
    d_dev, w_dev = [dev(d) for d in deltas], dev(w)
    out = torch.empty(rows, width, device="cuda", dtype=DT[dtype])
    small_in = dev(torch.randn(1, 64, generator=g).to(DT[dtype]))
    small_out = torch.empty(1, 32, device="cuda", dtype=DT[dtype])
    total = stream.double() + sum(d.double() for d in deltas)
    for between in (False, True):
        for _ in range(5):
            s = dev(stream.clone())
            for d in d_dev:
                ops().add_rmsnorm(s, d, w_dev, out, eps)
                if between:
                    ops().swiglu(small_in, small_out)
            close(s, total, "float32")
            close(out, plain.rms_norm(total, w.double(), eps), dtype)


@pytest.mark.parametrize("dtype", list(DT))
def test_rmsnorm_on_head_vectors(dtype):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(11, 5, 48, generator=g).to(DT[dtype])
    w = 1 + 0.1 * torch.randn(48, generator=g)
    out = torch.empty_like(dev(x))
    ops().rmsnorm(dev(x), dev(w), out, 1e-6)
    close(out, plain.rms_norm(x.double(), w.double(), 1e-6), dtype)


@pytest.mark.parametrize("shape", [(37, 70, 53), (1, 331, 96), (130, 64, 200), (64, 64, 16)])
def test_gemm_f32_is_true_float32(shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(3)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = torch.empty(M, N, device="cuda")
    ops().gemm_f32_nt(dev(a), dev(w), out)
    want = a.double() @ w.double().t()
    # float32 FMA chain over K terms: error ~ K * 2^-24 of the row's magnitude, far below TF32's 2^-11
    assert float((out.cpu().double() - want).abs().max()) <= 1e-6 * K ** 0.5 * float(want.abs().max())
    # rows do not depend on the other rows of the batch
    one = torch.empty(1, N, device="cuda")
    ops().gemm_f32_nt(dev(a[M // 2:M // 2 + 1].contiguous()), dev(w), one)
    assert torch.equal(one[0], out[M // 2])


@pytest.mark.parametrize("dtype", list(DT))
def test_swiglu(dtype):
    g = torch.Generator().manual_seed(4)
    gu = (torch.randn(19, 400, generator=g) * 3).to(DT[dtype])
    out = torch.empty(19, 200, device="cuda", dtype=DT[dtype])
    ops().swiglu(dev(gu), out)
    gate, up = gu[:, :200].double(), gu[:, 200:].double()
    close(out, up * gate * torch.sigmoid(gate), dtype)


@pytest.mark.parametrize("shape", [(1, 4096, 1024), (8, 1024, 2048), (16, 331, 96), (3, 70, 200), (9, 48, 8),
                                   (5, 151936, 64), (16, 16, 3072), (7, 1024, 3072), (3, 1000, 2056), (2, 64, 5000),
                                   # tens of megabytes of weights, K split over 1, 2, 4 and 8 warps, ragged ends
                                   (3, 6144, 4096), (8, 9000, 1400), (1, 2328, 5448), (7, 600, 20488), (2, 4736, 2648)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_gemm_skinny(shape, out_dtype):
    T, N, K = shape
    g = torch.Generator().manual_seed(8)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    out = torch.full((T, N), float("nan"), device="cuda", dtype=DT[out_dtype])
    ops().gemm_skinny(dev(x), dev(w), out)
    want = x.double() @ w.double().t()
    close(out, want, out_dtype, scale=float(want.abs().max()),
          tol=f32_accumulation_tol(K) if out_dtype == "float32" else None)
    assert ops().gemm_skinny_takes(T, dev(w)) and not ops().gemm_skinny_takes(17, dev(w))


@pytest.mark.parametrize("shape", [(1, 3072, 1024), (8, 136, 96), (13, 200, 80), (5, 12288, 1024), (8, 3000, 4104)])
def test_gemm_skinny_with_swiglu(shape):
    T, inter, K = shape
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g) * 0.2).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.cat([gate.view(inter // 8, 8, K), up.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    out = torch.full((T, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops().gemm_skinny(dev(x), dev(w), out, swiglu_blocks=True)
    gv, uv = x.double() @ gate.double().t(), x.double() @ up.double().t()
    want = uv * gv * torch.sigmoid(gv)
    close(out, want, "bfloat16")
    # the unfused pair (library product + gate kernel on the same layout) agrees
    gu = (x.float() @ w.float().t()).to(torch.bfloat16)
    out2 = torch.empty_like(out)
    ops().swiglu(dev(gu), out2, interleave8=True)
    close(out2, want, "bfloat16", scale=float(want.abs().max()) * 2)


@pytest.mark.parametrize("shape", [(1, 4096, 1024), (8, 1024, 2048), (16, 331, 96), (3, 70, 200), (9, 48, 8), (7, 1024, 3072),
                                   (5, 64, 5000), (12, 1024, 2048), (16, 1024, 3072), (10, 2368, 2048),
                                   (4, 4096, 4096), (8, 5120, 8192), (1, 1000, 12296)])
def test_gemm_skinny_into_stream(shape):
    """stream += x W^T in place, with partial sums of squares of the new rows that add up to the rows' own."""
    T, N, K = shape
    g = torch.Generator().manual_seed(31)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    stream = torch.randn(T, N, generator=g) * 3
    s = dev(stream.clone())
    parts = ops().sumsq_parts(N)
    sums = torch.full((parts + 1, ops().SUMSQ_ROWS), float("nan"), device="cuda")
    next_w = 1 + 0.3 * torch.randn(N, generator=g)
    scaled = torch.full((T, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    for _ in range(2):  # the second call runs right after a launch that wrote a stream
        s.copy_(dev(stream))
        assert ops().gemm_skinny_into_stream(dev(x), dev(w), s, sums) == parts
    s.copy_(dev(stream))
    assert ops().gemm_skinny_into_stream(dev(x), dev(w), s, sums, dev(next_w), scaled) == parts
    # the new rows times the next norm's weight, rounded once
    assert torch.equal(scaled.cpu(), (s.cpu() * next_w).to(torch.bfloat16))
    want = stream.double() + x.double() @ w.double().t()
    close(s, want, "float32", scale=float(want.abs().max()), tol=f32_accumulation_tol(K))
    got = sums[:parts, :T].double().sum(0).cpu()
    assert torch.allclose(got, (s.cpu().double() ** 2).sum(1), rtol=1e-5)
    assert torch.isnan(sums[parts]).all()


@pytest.mark.parametrize("shape", [(1, 4096, 1024), (8, 6144, 1024), (16, 331, 96), (3, 70, 200), (9, 48, 8), (6, 64, 5000),
                                   (12, 2048, 4096), (8, 1024, 5120), (8, 6144, 4096), (3, 24576, 1024), (2, 2400, 5120)])
@pytest.mark.parametrize("with_swiglu", [False, True])
def test_gemm_skinny_normed(shape, with_swiglu):
    """rmsnorm(stream) W^T without a norm kernel: the operand is the stream times the norm weight in bfloat16,
    and 1 / rms is applied after the product, from partial sums of squares, both laid out as
    gemm_skinny_into_stream leaves them."""
    T, N, K = shape
    if with_swiglu:
        N = N // 16 * 16
    g = torch.Generator().manual_seed(32)
    eps = 1e-5
    stream = torch.randn(T, K, generator=g) * 4
    nw = 1 + 0.2 * torch.randn(K, generator=g)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    parts = ops().sumsq_parts(K)  # one partial sum per 16 columns of the stream, row pitch 16
    sq = torch.zeros(parts, ops().SUMSQ_ROWS)
    padded = torch.zeros(T, parts * 16)
    padded[:, :K] = stream
    sq[:, :T] = (padded.view(T, parts, 16) ** 2).sum(2).t()
    scaled = (stream * nw).to(torch.bfloat16)
    out = torch.full((T, N // 2 if with_swiglu else N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops().gemm_skinny_normed(dev(scaled), dev(sq), parts, eps, dev(w), out, swiglu_blocks=with_swiglu)
    # what the kernel is specified to compute: the product of the rounded operand, then 1 / rms; against the
    # plain norm followed by the product it differs by where the one rounding of the activations falls
    rs = 1.0 / torch.sqrt((stream.double() ** 2).mean(1, keepdim=True) + eps)
    want = (scaled.double() @ w.double().t()) * rs
    loose = plain.rms_norm(stream.double(), nw.double(), eps) @ w.double().t()
    assert float((want - loose).abs().max()) <= 4e-3 * float(loose.abs().max())
    if with_swiglu:
        gate = want.view(T, N // 16, 2, 8)[:, :, 0].reshape(T, N // 2)
        up = want.view(T, N // 16, 2, 8)[:, :, 1].reshape(T, N // 2)
        want = up * gate * torch.sigmoid(gate)
    close(out, want, "bfloat16")


@pytest.mark.parametrize("shape", [(128, 128, 64), (2048, 4096, 1024), (100, 200, 72), (257, 331, 96), (1, 64, 8),
                                   (300, 1024, 3072)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("pair", [False, True])
def test_gemm_tc(shape, out_dtype, pair):
    """The tcgen05 / TMA product at sizes that do and do not fill its tiles, by single CTAs (128 x 128 or 256
    x 64) and by pairs of CTAs with the paired instruction (256 x 256 x 64)."""
    M, N, K = shape
    g = torch.Generator().manual_seed(10)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[out_dtype])
    st = status()
    ops().gemm_tc(dev(x), dev(w), out, st, pair=pair)
    assert int(st.item()) == 0
    want = x.double() @ w.double().t()
    close(out, want, out_dtype, scale=float(want.abs().max()),
          tol=f32_accumulation_tol(K) if out_dtype == "float32" else None)


@pytest.mark.parametrize("shape", [(128, 3072, 1024), (300, 136, 96), (2048, 200, 80), (1300, 1000, 2048)])
@pytest.mark.parametrize("pair", [False, True])
def test_gemm_tc_with_swiglu(shape, pair):
    T, inter, K = shape
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g) * 0.2).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.cat([gate.view(inter // 8, 8, K), up.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    out = torch.full((T, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    st = status()
    ops().gemm_tc(dev(x), dev(w), out, st, swiglu_blocks=True, pair=pair)
    assert int(st.item()) == 0
    gv, uv = x.double() @ gate.double().t(), x.double() @ up.double().t()
    close(out, uv * gv * torch.sigmoid(gv), "bfloat16")


def paged(kv, page_size, tables, num_pages, dtype):
    """Scatters per-request [len, Hkv, D] keys (or values) into pages [P, Hkv, page, D] (NaN elsewhere)."""
    hkv, d = kv[0].shape[1:]
    pages = torch.full((num_pages, hkv, page_size, d), float("nan"))
    for seq, table in zip(kv, tables):
        for pos in range(seq.shape[0]):
            pages[table[pos // page_size], :, pos % page_size] = seq[pos]
    return pages.to(dtype)


def make_tables(lengths, page_size, seed, extra=3):
    """Block tables that are scattered and partly reversed, to prove the indirection."""
    need = [-(-n // page_size) for n in lengths]
    num_pages = sum(need) + extra
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    tables, at = [], 0
    for n in need:
        tables.append(perm[at:at + n][::-1])
        at += n
    return tables, num_pages


def table_tensor(tables):
    stride = max(len(t) for t in tables)
    return torch.tensor([t + [-1] * (stride - len(t)) for t in tables], dtype=torch.int32)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("with_table", [False, True])
@pytest.mark.parametrize("hq,hkv,d,rot", [(6, 3, 48, 48), (4, 1, 80, 32), (8, 2, 128, 128), (2, 2, 16, 16),
                                          (3, 1, 64, 64), (5, 1, 32, 32), (3, 2, 256, 256), (16, 8, 128, 128)])
def test_qkv_post(dtype, hq, hkv, d, rot, with_table):
    """Head norm + rotation + scatter, with a partial rotary width and pages out of order; with the
    angles computed in the kernel and with the step's table of sines and cosines."""
    g = torch.Generator().manual_seed(5)
    page_size, eps, theta = 8, 1e-6, 10000.0
    starts, news = [0, 13, 40], [21, 1, 7]  # tokens already cached, tokens of this step
    lengths = [s + n for s, n in zip(starts, news)]
    tables, num_pages = make_tables(lengths, page_size, 6)
    T = sum(news)
    qkv = torch.randn(T, (hq + 2 * hkv) * d, generator=g).to(DT[dtype])
    qw, kw = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.tensor([s + i for s, n in zip(starts, news) for i in range(n)], dtype=torch.int32)
    tok_seq = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    k_pages = torch.zeros(num_pages, hkv, page_size, d, device="cuda", dtype=DT[dtype])
    v_pages = torch.zeros_like(k_pages)
    q_out = torch.empty(T, hq, d, device="cuda", dtype=DT[dtype])
    st = status()
    cos_sin = None
    if with_table:
        cos_sin = torch.empty(T, rot, device="cuda", dtype=torch.float32)
        ops().rope_table(dev(inv_freq), dev(positions), cos_sin)
        ang32 = positions.float()[:, None] * inv_freq[None, :]
        assert torch.allclose(cos_sin.cpu(), torch.cat([ang32.cos(), ang32.sin()], dim=1), atol=2e-6)
    ops().qkv_post(dev(qkv), q_out, k_pages, v_pages, dev(qw), dev(kw), eps, dev(inv_freq), rot, dev(positions),
                   dev(tok_seq), dev(table_tensor(tables)), hq, hkv, d, True, st, cos_sin=cos_sin)
    assert int(st.item()) == 0
    x = qkv.double().view(T, hq + 2 * hkv, d)
    q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
    q, k = plain.rms_norm(q, qw.double(), eps), plain.rms_norm(k, kw.double(), eps)
    ang = positions.double()[:, None] * inv_freq.double()[None, :]
    cos, sin = ang.cos(), ang.sin()

    def rotate(t):
        out = t.clone()
        out[..., :rot] = plain.apply_rope(t[..., :rot], cos, sin)
        return out

    q, k = rotate(q), rotate(k)
    close(q_out, q, dtype)
    kp, vp = k_pages.cpu().double(), v_pages.cpu().double()
    for t in range(T):
        page = tables[int(tok_seq[t])][int(positions[t]) // page_size]
        slot = int(positions[t]) % page_size
        close(kp[page, :, slot], k[t], dtype, scale=float(k.abs().max()))
        close(vp[page, :, slot], v[t], dtype, scale=float(v.abs().max()))
    # nothing else was written
    written = torch.zeros(num_pages, page_size, dtype=torch.bool)
    for t in range(T):
        written[tables[int(tok_seq[t])][int(positions[t]) // page_size], int(positions[t]) % page_size] = True
    assert float(kp.abs().sum(dim=(1, 3))[~written].sum()) == 0.0
    # a page id outside the pool is reported, not written
    bad = table_tensor(tables)
    bad[0, 0] = num_pages
    ops().qkv_post(dev(qkv), q_out, k_pages, v_pages, dev(qw), dev(kw), eps, dev(inv_freq), rot, dev(positions),
                   dev(tok_seq), dev(bad), hq, hkv, d, True, st, cos_sin=cos_sin)
    assert int(st.item()) & 2


@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("hq,hkv,d,K,T", [(8, 2, 128, 256, 200), (5, 2, 128, 96, 130), (3, 1, 64, 136, 333),
                                          (16, 8, 128, 1024, 256), (16, 8, 128, 512, 1100), (6, 1, 64, 72, 2500)])
def test_gemm_tc_qkv(hq, hkv, d, K, T, rotate, pair):
    """The QKV projection with head norm, rotation and cache write in its epilogue against the plain
    formulas applied to the projection rounded to bfloat16; rows and heads that do not fill a tile."""
    g = torch.Generator().manual_seed(13)
    page_size, eps, theta = 16, 1e-6, 10000.0
    starts, news = [5, 0], [T - 40, 40]
    lengths = [s + n for s, n in zip(starts, news)]
    tables, num_pages = make_tables(lengths, page_size, 4)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn((hq + 2 * hkv) * d, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    qw, kw = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.tensor([s + i for s, n in zip(starts, news) for i in range(n)], dtype=torch.int32)
    tok_seq = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    k_pages = torch.zeros(num_pages, hkv, page_size, d, device="cuda", dtype=torch.bfloat16)
    v_pages = torch.zeros_like(k_pages)
    q_out = torch.full((T, hq, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    st = status()
    cos_sin = None
    if rotate:
        cos_sin = torch.empty(T, d, device="cuda", dtype=torch.float32)
        ops().rope_table(dev(inv_freq), dev(positions), cos_sin)
    assert ops().gemm_tc_qkv_takes(T, dev(x), dev(w), d, d if rotate else 0)
    ops().gemm_tc_qkv(dev(x), dev(w), q_out, k_pages, v_pages, dev(qw), dev(kw), eps, cos_sin, dev(positions),
                      dev(tok_seq), dev(table_tensor(tables)), hq, hkv, d, True, st, pair=pair)
    assert int(st.item()) == 0
    qkv = (x.double() @ w.double().t()).to(torch.bfloat16).double().view(T, hq + 2 * hkv, d)
    q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
    q, k = plain.rms_norm(q, qw.double(), eps), plain.rms_norm(k, kw.double(), eps)
    if rotate:
        ang = positions.double()[:, None] * inv_freq.double()[None, :]
        q, k = plain.apply_rope(q, ang.cos(), ang.sin()), plain.apply_rope(k, ang.cos(), ang.sin())
    # The projection is rounded to bfloat16 before the norm.  Where float32 accumulation (the kernel) and
    # the exact product (here) fall on different sides of a rounding boundary, the norm's input differs
    # by one bfloat16 step, 2^-8 relative; with the 2^-9 of the output's own rounding: 1.5 * 2^-8.
    flip_tol = 1.5 * 2.0 ** -8
    close(q_out, q, "bfloat16", tol=flip_tol)
    kp, vp = k_pages.cpu().double(), v_pages.cpu().double()
    for t in range(T):
        page = tables[int(tok_seq[t])][int(positions[t]) // page_size]
        slot = int(positions[t]) % page_size
        close(kp[page, :, slot], k[t], "bfloat16", scale=float(k.abs().max()), tol=flip_tol)
        close(vp[page, :, slot], v[t], "bfloat16", scale=float(v.abs().max()))
    written = torch.zeros(num_pages, page_size, dtype=torch.bool)
    for t in range(T):
        written[tables[int(tok_seq[t])][int(positions[t]) // page_size], int(positions[t]) % page_size] = True
    assert float(kp.abs().sum(dim=(1, 3))[~written].sum()) == 0.0


@pytest.mark.parametrize("pair", [False, True])
def test_gemm_tc_qkv_without_head_norm_and_without_a_cache_write(pair):
    """The same epilogue for a layer without head norms that reads a cache another layer wrote: only q is
    produced (rotated), the pages stay as they are; and a page id outside the pool is reported, not written."""
    g = torch.Generator().manual_seed(14)
    hq, hkv, d, K, T, page_size = 6, 2, 128, 192, 150, 16
    tables, num_pages = make_tables([T], page_size, 5)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn((hq + 2 * hkv) * d, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    positions = torch.arange(T, dtype=torch.int32)
    tok_seq = torch.zeros(T, dtype=torch.int32)
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    k_pages = torch.full((num_pages, hkv, page_size, d), 3.0, device="cuda", dtype=torch.bfloat16)
    v_pages = torch.full_like(k_pages, 5.0)
    q_out = torch.full((T, hq, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    cos_sin = torch.empty(T, d, device="cuda", dtype=torch.float32)
    ops().rope_table(dev(inv_freq), dev(positions), cos_sin)
    st = status()
    ops().gemm_tc_qkv(dev(x), dev(w), q_out, k_pages, v_pages, None, None, 0.0, cos_sin, dev(positions), dev(tok_seq),
                      dev(table_tensor(tables)), hq, hkv, d, False, st, pair=pair)
    assert int(st.item()) == 0
    q = (x.double() @ w.double().t()).to(torch.bfloat16).double().view(T, hq + 2 * hkv, d)[:, :hq]
    ang = positions.double()[:, None] * inv_freq.double()[None, :]
    close(q_out, plain.apply_rope(q, ang.cos(), ang.sin()), "bfloat16", tol=1.5 * 2.0 ** -8)
    assert bool((k_pages == 3.0).all()) and bool((v_pages == 5.0).all())
    bad = table_tensor(tables)
    bad[0, 2] = num_pages
    ops().gemm_tc_qkv(dev(x), dev(w), q_out, k_pages, v_pages, None, None, 0.0, cos_sin, dev(positions), dev(tok_seq),
                      dev(bad), hq, hkv, d, True, st, pair=pair)
    assert int(st.item()) & 2
    hit = [p for p in range(num_pages) if p != tables[0][2] and p in tables[0]]
    assert bool((k_pages[tables[0][2]] == 3.0).all()), "the rows of the bad page went somewhere"
    assert not bool((k_pages[hit] == 3.0).all())


def reference_attention(q, k_list, v_list, q_lens, window):
    """Per request: the plain whole-sequence attention, of which the last q_len rows are the step's."""
    outs = []
    at = 0
    for k, v, n in zip(k_list, v_list, q_lens):
        total = k.shape[0]
        full_q = torch.zeros(total, q.shape[1], q.shape[2], dtype=q.dtype)
        full_q[total - n:] = q[at:at + n]
        outs.append(plain.causal_attention(full_q, k, v, window)[total - n:])
        at += n
    return torch.cat(outs)


def attention_case(dtype, hq, hkv, d, page_size, kv_lens, q_lens, window, seed=7, kernel="attn_ref"):
    g = torch.Generator().manual_seed(seed)
    tables, num_pages = make_tables(kv_lens, page_size, seed + 1)
    k_list = [torch.randn(n, hkv, d, generator=g).to(DT[dtype]) for n in kv_lens]
    v_list = [torch.randn(n, hkv, d, generator=g).to(DT[dtype]) for n in kv_lens]
    T = sum(q_lens)
    q = torch.randn(T, hq, d, generator=g).to(DT[dtype])
    return q, k_list, v_list, tables, num_pages


def run_attention(kernel, q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window, dtype):
    k_pages = dev(paged(k_list, page_size, tables, num_pages, DT[dtype]))
    v_pages = dev(paged(v_list, page_size, tables, num_pages, DT[dtype]))
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    tok_seq = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32)
    out = torch.empty_like(dev(q))
    st = status()
    scale = q.shape[-1] ** -0.5
    getattr(ops(), kernel)(dev(q), k_pages, v_pages, out, dev(q_start), dev(torch.tensor(kv_lens, dtype=torch.int32)),
                           dev(tok_seq), dev(table_tensor(tables)), scale, window or 0, st)
    assert int(st.item()) == 0
    return out


ATTN_SHAPES = [
    # hq, hkv, d, page, kv_lens, q_lens, window
    (6, 3, 48, 8, [21, 14, 47], [21, 1, 7], None),      # whole prompt, one decoded token, a portion
    (4, 1, 80, 16, [100, 3, 33], [2, 3, 1], None),      # ragged, two-token portion, head size 80
    (8, 2, 128, 16, [300, 129], [1, 1], None),          # decode over hundreds of keys
    (4, 2, 16, 4, [50, 9], [50, 2], 12),                # window shorter than the sequence
    (5, 5, 32, 8, [64, 41], [5, 41], 8),                # window = page, no grouping
    (16, 8, 64, 16, [17], [17], 1000),                  # window longer than the sequence
]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("case", ATTN_SHAPES)
def test_attn_ref(dtype, case):
    hq, hkv, d, page_size, kv_lens, q_lens, window = case
    q, k_list, v_list, tables, num_pages = attention_case(dtype, hq, hkv, d, page_size, kv_lens, q_lens, window)
    out = run_attention("attn_ref", q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window, dtype)
    want = reference_attention(q.double(), [k.double() for k in k_list], [v.double() for v in v_list], q_lens, window)
    close(out, want, dtype)


@pytest.mark.parametrize("d,page_size,hq,hkv", [(128, 16, 16, 8), (64, 32, 6, 2), (128, 64, 4, 4)])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("with_norm", [True, False])
@pytest.mark.parametrize("many", [False, True])
def test_decode_attention_from_the_raw_projection(d, page_size, hq, hkv, splits, window, with_norm, many):
    """A step of single tokens: the decode kernel norms and rotates its query and the new key itself and stores
    the new key and value, against qkv_post followed by the same kernel.  Lengths that put the new token at
    the start, in the middle and at the end of a tile and of a page.  ``many``: seventy more sequences, so that
    the grid has more blocks than three per SM hold and the kernel's form for four per SM runs."""
    if many and ((d, hkv) != (128, 8) or not with_norm):
        pytest.skip("the large grid is run at one shape")
    o = ops()
    kv_lens = [200, 17, 161, 1, 16, 64, 65] + ([18 + (37 * i) % 190 for i in range(70)] if many else [])
    B, n_heads, eps = len(kv_lens), hq + 2 * hkv, 1e-5
    g = torch.Generator().manual_seed(41)
    q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, [1] * B, window, seed=23)
    qkv = (torch.randn(B, n_heads * d, generator=g) * 2).to(torch.bfloat16)
    qw = (1 + 0.2 * torch.randn(d, generator=g)) if with_norm else None
    kw = (1 + 0.2 * torch.randn(d, generator=g)) if with_norm else None
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    positions = torch.tensor([n - 1 for n in kv_lens], dtype=torch.int32)
    table_dev = dev(table_tensor(tables))
    cos_sin = torch.empty(B, d, device="cuda")
    o.rope_table(dev(inv_freq), dev(positions), cos_sin)
    q_start = dev(torch.arange(B + 1, dtype=torch.int32))
    tok_seq = dev(torch.arange(B, dtype=torch.int32))
    lens = dev(torch.tensor(kv_lens, dtype=torch.int32))
    partial = torch.empty(o.decode_partial_numel(B, hq, d), device="cuda")
    scale = d ** -0.5

    def pools():  # the row of the new token holds NaN until somebody writes it
        kl = [k.clone() for k in k_list]
        vl = [v.clone() for v in v_list]
        for k, v in zip(kl, vl):
            k[-1] = float("nan")
            v[-1] = float("nan")
        return (dev(paged(kl, page_size, tables, num_pages, torch.bfloat16)),
                dev(paged(vl, page_size, tables, num_pages, torch.bfloat16)))

    # two kernels
    k1, v1 = pools()
    q1 = torch.empty(B, hq, d, device="cuda", dtype=torch.bfloat16)
    st = status()
    o.qkv_post(dev(qkv), q1, k1, v1, None if qw is None else dev(qw), None if kw is None else dev(kw), eps, dev(inv_freq), d,
               dev(positions), tok_seq, table_dev, hq, hkv, d, True, st, cos_sin=cos_sin)
    out1 = torch.full((B, hq, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    o.attn_decode(q1, k1, v1, out1, partial, q_start, lens, table_dev, B, scale, window or 0, splits, st, loader="tma")
    # one kernel
    k2, v2 = pools()
    out2 = torch.full_like(out1, float("nan"))
    raw = (dev(qkv), None if qw is None else dev(qw), None if kw is None else dev(kw), eps, cos_sin, True)
    o.attn_decode(q1, k2, v2, out2, partial, q_start, lens, table_dev, B, scale, window or 0, splits, st, loader="tma",
                  raw_qkv=raw)
    assert int(st.item()) == 0
    # the same formulas in the same precision; the sums of squares are added in another order, which may move
    # a value by one bfloat16 step (2^-8 relative) before the attention
    used = ~torch.isnan(k1.float())
    assert torch.equal(used, ~torch.isnan(k2.float())) and torch.equal(~torch.isnan(v1.float()), ~torch.isnan(v2.float()))
    assert torch.equal(v1[used], v2[used])
    kd = (k1[used].float() - k2[used].float()).abs()
    assert float(kd.max()) <= 2.0 ** -7 * float(k1[used].float().abs().max())
    close(out2, out1, "bfloat16")
    # and without writing (a layer that reads a cache another layer wrote): the pools stay as they are
    k3, v3 = pools()
    before_k, before_v = k3.clone(), v3.clone()
    out3 = torch.full_like(out1, float("nan"))
    o.attn_decode(q1, k3, v3, out3, partial, q_start, lens, table_dev, B, scale, window or 0, splits, st, loader="tma",
                  raw_qkv=raw[:5] + (False,))
    assert torch.equal(torch.nan_to_num(k3.float(), 7.0), torch.nan_to_num(before_k.float(), 7.0))
    assert torch.equal(torch.nan_to_num(v3.float(), 7.0), torch.nan_to_num(before_v.float(), 7.0))


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("far", [0, 3, 250, 511])
def test_attn_ref_finds_one_far_key(dtype, far):
    """Among 512 random keys one is made to match the query strongly: the output must be that
    key's value, whichever page it lies in (random weights alone would average everything)."""
    hq, hkv, d, page_size = 4, 2, 64, 16
    kv_lens, q_lens = [512], [1]
    q, k_list, v_list, tables, num_pages = attention_case(dtype, hq, hkv, d, page_size, kv_lens, q_lens, None, seed=11)
    q = (q.float() * 0 + 1.0).to(DT[dtype])
    k_list[0] = (k_list[0].float() * 0.05).to(DT[dtype])
    k_list[0][far] = 4.0  # score 4 * 64 / 8 = 32 against ~0 for the rest
    out = run_attention("attn_ref", q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, None, dtype)
    want = v_list[0][far].double()  # [hkv, d]
    got = out.cpu().double().view(hq, d)
    for h in range(hq):
        assert float((got[h] - want[h // 2]).abs().max()) < 1e-2


def test_attn_ref_window_edge_is_exact():
    """The key just outside the window carries a huge value: any off-by-one shows at once."""
    hq, hkv, d, page_size, window = 2, 1, 32, 8, 10
    kv_lens, q_lens = [40], [40]
    q, k_list, v_list, tables, num_pages = attention_case("float32", hq, hkv, d, page_size, kv_lens, q_lens, window, seed=13)
    out0 = run_attention("attn_ref", q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window, "float32")
    want = reference_attention(q.double(), [k_list[0].double()], [v_list[0].double()], q_lens, window)
    close(out0, want, "float32")
    # poisoning a value outside every query's window from position 25 on changes nothing there
    v_list[0][10] = 1e6
    out1 = run_attention("attn_ref", q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window, "float32")
    assert torch.equal(out0[20:], out1[20:])      # queries 20.. see keys 11.. only
    assert not torch.equal(out0[19], out1[19])    # query 19 still sees key 10


def run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window, splits=None,
             portion_kernel="auto", loader="cp_async"):
    """The tensor-core kernels through the dispatcher (or the decode kernel with a forced split count).
    Unused slots of the pages hold NaN: anything read past a sequence's keys poisons the result."""
    o = ops()
    k_pages = dev(paged(k_list, page_size, tables, num_pages, torch.bfloat16))
    v_pages = dev(paged(v_list, page_size, tables, num_pages, torch.bfloat16))
    order = sorted(range(len(q_lens)), key=lambda i: (q_lens[i] != 1, i))  # single-token rows first
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    q_sorted = torch.cat([q[starts[i]:starts[i + 1]] for i in order])
    ql = [q_lens[i] for i in order]
    kl = [kv_lens[i] for i in order]
    tb = [tables[i] for i in order]
    q_start = torch.tensor([0] + list(torch.tensor(ql).cumsum(0)), dtype=torch.int32)
    tok_seq = torch.tensor([b for b, n in enumerate(ql) for _ in range(n)], dtype=torch.int32)
    num_decode = sum(1 for n in ql if n == 1)
    hq, d = q.shape[1], q.shape[2]
    partial = torch.empty(o.decode_partial_numel(len(ql), hq, d), device="cuda")
    out = torch.full_like(dev(q_sorted), float("nan"))
    st = status()
    scale = d ** -0.5
    args = (dev(q_sorted), k_pages, v_pages, out)
    if splits is None:
        o.paged_attention(*args, dev(q_start), dev(torch.tensor(kl, dtype=torch.int32)), dev(tok_seq),
                          dev(table_tensor(tb)), len(ql), num_decode, max(ql), max(kl), scale, window or 0, st, partial,
                          portion_kernel=portion_kernel,
                          decode_kernel="cp_async" if portion_kernel == "mma" else "auto")
    else:
        assert num_decode == len(ql)
        o.attn_decode(*args, partial, dev(q_start), dev(torch.tensor(kl, dtype=torch.int32)), dev(table_tensor(tb)),
                      len(ql), scale, window or 0, splits, st, loader=loader)
    assert int(st.item()) == 0
    # back to the caller's order
    pieces, at = {}, 0
    for i, n in zip(order, ql):
        pieces[i] = out[at:at + n]
        at += n
    return torch.cat([pieces[i] for i in range(len(q_lens))])


FAST_SHAPES = ATTN_SHAPES + [
    (16, 8, 128, 16, [700, 65, 1, 333], [1, 1, 1, 1], None),     # decode, the engine's big head size
    (16, 8, 128, 16, [700, 65, 130], [700, 64, 3], None),        # whole prompts and portions at head size 128
    (8, 1, 64, 16, [200, 90], [40, 90], None),                   # eight heads to one kv head
    (32, 2, 16, 4, [37], [5], None),                             # sixteen heads to one kv head, page of 4
    (6, 2, 96, 8, [129, 64], [129, 1], 33),                      # head size 96, window across tiles
    (4, 2, 256, 16, [150, 20], [22, 1], None),                   # largest head size
    (3, 1, 112, 16, [77, 300], [77, 1], 100),                    # three heads to one kv head
]


FAST_SHAPES += [
    (16, 8, 128, 16, [2048], [2048], None),                      # a whole long prompt: many key tiles per query tile
    (4, 2, 64, 8, [333, 64, 191], [100, 64, 191], None),          # head size 64, pages of 8, ragged ends
    (8, 4, 128, 32, [500, 70], [37, 70], None),                   # pages of 32
    (2, 1, 128, 64, [129], [129], None),                          # pages of 64
]


@pytest.mark.parametrize("portion_kernel", ["auto", "mma"])
@pytest.mark.parametrize("case", FAST_SHAPES)
def test_fast_attention_against_plain(case, portion_kernel):
    """``auto`` sends portions to the tcgen05 kernel where it takes the shape (head 64 / 128, pages of
    8..64, no window) and to the mma.sync kernel otherwise; ``mma`` tests the latter on every shape."""
    hq, hkv, d, page_size, kv_lens, q_lens, window = case
    q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, q_lens, window)
    out = run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window,
                   portion_kernel=portion_kernel)
    want = reference_attention(q.double(), [k.double() for k in k_list], [v.double() for v in v_list], q_lens, window)
    # probabilities are rounded to bfloat16 before P.V (as the reference does) and so is the output:
    # two roundings of 2^-9 each
    close(out, want, "bfloat16", scale=None)


@pytest.mark.parametrize("loader,d,page_size", [("cp_async", 64, 16), ("tma", 64, 16), ("tma", 128, 32),
                                                ("cp_async", 48, 8)])
@pytest.mark.parametrize("splits", [1, 2, 3, 4, 7, 12, 31, 32])
@pytest.mark.parametrize("window", [None, 150])
def test_decode_splits_agree(splits, window, loader, d, page_size):
    hq, hkv = 8, 2
    kv_lens, q_lens = [1000, 17, 160, 1, 16], [1, 1, 1, 1, 1]
    q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, q_lens, window, seed=21)
    out = run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window, splits=splits,
                   loader=loader)
    want = reference_attention(q.double(), [k.double() for k in k_list], [v.double() for v in v_list], q_lens, window)
    close(out, want, "bfloat16")


@pytest.mark.parametrize("splits", [None, 2, 5])
@pytest.mark.parametrize("hq,hkv,d,page_size", [(8, 4, 128, 16), (6, 2, 64, 32)])
def test_decode_of_many_sequences(splits, hq, hkv, d, page_size):
    """More (sequence, kv head, range) blocks than the SMs hold at once, so that the grid runs in several waves;
    ragged lengths, some of them shorter than a range."""
    g = torch.Generator().manual_seed(31)
    n = 130 if hkv == 4 else 260
    kv_lens = [int(x) for x in torch.randint(1, 420, (n,), generator=g)]
    kv_lens[3], kv_lens[17] = 1, 16
    q_lens = [1] * n
    q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, q_lens, None, seed=33)
    out = run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, None, splits=splits, loader="tma")
    want = reference_attention(q.double(), [k.double() for k in k_list], [v.double() for v in v_list], q_lens, None)
    close(out, want, "bfloat16")


@pytest.mark.parametrize("far", [0, 3, 250, 511])
@pytest.mark.parametrize("q_len", [1, 6])
def test_fast_attention_finds_one_far_key(far, q_len):
    hq, hkv, d, page_size = 4, 2, 64, 16
    kv_lens, q_lens = [512 + q_len - 1], [q_len]
    q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, q_lens, None, seed=11)
    q = (q.float() * 0 + 1.0).to(torch.bfloat16)
    k_list[0] = (k_list[0].float() * 0.05).to(torch.bfloat16)
    k_list[0][far] = 4.0
    out = run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, None)
    want = v_list[0][far].double()
    got = out.cpu().double()
    for h in range(hq):
        assert float((got[:, h] - want[h // 2]).abs().max()) < 2e-2


def test_fast_attention_window_edge():
    hq, hkv, d, page_size, window = 2, 1, 32, 8, 10
    kv_lens, q_lens = [140], [140]
    q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, q_lens, window, seed=13)
    out0 = run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window)
    v_list[0][70] = 3e4  # visible to queries 70..79 only
    out1 = run_fast(q, k_list, v_list, tables, num_pages, page_size, kv_lens, q_lens, window)
    changed = [(out0[i] != out1[i]).any().item() for i in range(140)]
    assert changed == [70 <= i <= 79 for i in range(140)]
    # and one decoded token at the edge
    for length, sees in ((80, True), (81, False)):
        kv, ql = [length], [1]
        q1, kl, vl, tb, npg = attention_case("bfloat16", hq, hkv, d, page_size, kv, ql, window, seed=14)
        a = run_fast(q1, kl, vl, tb, npg, page_size, kv, ql, window)
        vl[0][70] = 3e4
        b2 = run_fast(q1, kl, vl, tb, npg, page_size, kv, ql, window)
        assert bool((a != b2).any()) == sees


def test_fast_attention_refuses_what_it_does_not_take():
    o = ops()
    assert not o.fast_attention_takes(torch.bfloat16, 4, 2, 24)
    assert not o.fast_attention_takes(torch.bfloat16, 34, 2, 64)
    assert not o.fast_attention_takes(torch.float32, 4, 2, 64)
    q = torch.zeros(1, 4, 24, device="cuda", dtype=torch.bfloat16)
    pages = torch.zeros(2, 2, 8, 24, device="cuda", dtype=torch.bfloat16)
    ints = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(o.KernelSizeError):
        o.attn_prefill(q, pages, pages, q.clone(), ints, ints, ints.view(1, 2), 1, 1, 1.0, 0, status())
    with pytest.raises(o.KernelSizeError):
        o.attn_decode(q, pages, pages, q.clone(), None, ints, ints, ints.view(1, 2), 1, 1.0, 0, 1, status())


@pytest.mark.parametrize("kernel", ["attn_ref_f32", "attn_ref_bf16", "decode_cp_async", "decode_tma", "attn_prefill",
                                    "attn_tc", "qkv_post_f32", "qkv_post_bf16", "decode_tma_raw"])
def test_a_length_beyond_the_block_table_is_flagged_and_not_read(kernel):
    """A request's length (or a token's position) one page beyond what the row pitch of the block table
    holds.  The first request's row is followed in memory by the second one's, whose entries are valid page
    ids: a kernel that indexed past the row's end would silently read (or, writing, overwrite) the other
    request's pages.  Every kernel must set the bad-position bit instead, touch no page it was not given,
    and leave finite output."""
    o = ops()
    bf16 = not kernel.endswith("f32")
    dtype = torch.bfloat16 if bf16 else torch.float32
    hq, hkv, d, page_size = 4, 2, 128 if bf16 else 48, 16
    g = torch.Generator().manual_seed(31)
    stride = 3                                   # pages a row of the table holds
    good_len = stride * page_size                # the longest length the table was made for
    bad_len = good_len + page_size               # one page beyond
    q_len = 1 if kernel.startswith(("decode", "attn_ref")) else 20
    num_pages = 2 * stride + 2
    table = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32)
    k_pages = dev(torch.randn(num_pages, hkv, page_size, d, generator=g).to(dtype))
    v_pages = dev(torch.randn(num_pages, hkv, page_size, d, generator=g).to(dtype))
    q = dev(torch.randn(2 * q_len, hq, d, generator=g).to(dtype))
    out = torch.zeros_like(q)
    q_start = dev(torch.tensor([0, q_len, 2 * q_len], dtype=torch.int32))
    tok_seq = dev(torch.tensor([0] * q_len + [1] * q_len, dtype=torch.int32))
    partial = torch.empty(o.decode_partial_numel(2, hq, d), device="cuda")
    scale = d ** -0.5

    def run(lengths):
        st = status()
        kv_len = dev(torch.tensor(lengths, dtype=torch.int32))
        if kernel.startswith("attn_ref"):
            o.attn_ref(q, k_pages, v_pages, out, q_start, kv_len, tok_seq, dev(table), scale, 0, st)
        elif kernel in ("decode_cp_async", "decode_tma"):
            o.attn_decode(q, k_pages, v_pages, out, partial, q_start, kv_len, dev(table), 2, scale, 0, 2, st,
                          loader=kernel[7:])
        elif kernel == "attn_prefill":
            o.attn_prefill(q, k_pages, v_pages, out, q_start, kv_len, dev(table), 2, q_len, scale, 0, st)
        elif kernel == "attn_tc":
            o.attn_tc(q, k_pages, v_pages, out, q_start, kv_len, dev(table), 2, q_len, scale, st)
        elif kernel.startswith("qkv_post") or kernel == "decode_tma_raw":
            T = 2 * q_len
            qkv = dev(torch.randn(T, (hq + 2 * hkv) * d, generator=g).to(dtype))
            positions = dev(torch.tensor([n - q_len + i for n in lengths for i in range(q_len)], dtype=torch.int32))
            before = (k_pages.clone(), v_pages.clone())
            if kernel == "decode_tma_raw":
                o.attn_decode(q, k_pages, v_pages, out, partial, q_start, kv_len, dev(table), 2, scale, 0, 2, st,
                              loader="tma", raw_qkv=(qkv, None, None, 0.0, None, True))
            else:
                o.qkv_post(qkv, out, k_pages, v_pages, None, None, 0.0, None, 0, positions, tok_seq, dev(table),
                           hq, hkv, d, True, st)
            # only slots of the tokens whose position the table covers may have changed
            allowed = torch.zeros(num_pages, page_size, dtype=torch.bool)
            for b, n in enumerate(lengths):
                for pos in range(n - q_len, n):
                    if pos // page_size < stride:
                        allowed[int(table[b, pos // page_size]), pos % page_size] = True
            for now, was in zip((k_pages, v_pages), before):
                changed = (now != was).any(dim=3).any(dim=1).cpu()
                assert not bool((changed & ~allowed).any()), "a slot outside the request's own pages was written"
            k_pages.copy_(before[0])
            v_pages.copy_(before[1])
        torch.cuda.synchronize()
        return int(st.item())

    assert run([good_len, good_len - 5]) == 0
    assert bool(torch.isfinite(out.float()).all())
    word = run([bad_len, good_len - 5])
    assert word & 4, f"status {word}: the bad-position bit is not set"
    assert bool(torch.isfinite(out.float()).all())
    with pytest.raises(o.KernelError):  # where the host knows the longest length it says so before any launch
        o.paged_attention(q, k_pages, v_pages, out, q_start, dev(torch.tensor([bad_len, 5], dtype=torch.int32)), tok_seq,
                          dev(table), 2, 2 if q_len == 1 else 0, q_len, bad_len, scale, 0, status(), partial)


def test_attn_tc_flags_more_new_tokens_than_the_request_holds():
    o = ops()
    hq, hkv, d, page_size = 4, 2, 128, 16
    q = torch.zeros(40, hq, d, device="cuda", dtype=torch.bfloat16)
    pages = torch.zeros(4, hkv, page_size, d, device="cuda", dtype=torch.bfloat16)
    st = status()
    o.attn_tc(q, pages, pages, q.clone(), dev(torch.tensor([0, 40], dtype=torch.int32)),
              dev(torch.tensor([30], dtype=torch.int32)), dev(torch.tensor([[0, 1, 2]], dtype=torch.int32)), 1, 40,
              d ** -0.5, st)
    assert int(st.item()) & 4


@pytest.mark.parametrize("kernel", ["gemm_tc", "gemm_tc_pair", "attn_tc", "attn_decode_tma", "attn_decode_tma_many"])
def test_a_wait_that_runs_out_is_given_up_cleanly(kernel):
    """The bounded waits of the TMA / tcgen05 kernels, made to run out: the loader is told to leave out one
    copy, so the barrier that copy would complete never does.  With the poll limit made small the kernel must
    return by itself with the time-out bit set, and the next ordinary launch of the same kernel (which needs
    the tensor memory and the barriers' shared memory that the abandoned blocks held) must give the right
    result.  No wait anywhere spins without a limit; nothing here faults."""
    o = ops()
    g = torch.Generator().manual_seed(77)
    if kernel.startswith("gemm_tc"):  # "gemm_tc_pair": both CTAs of a pair must give up, meet and free the pair's TMEM
        x = dev(torch.randn(256, 256, generator=g).to(torch.bfloat16))
        w = dev(torch.randn(384, 256, generator=g).to(torch.bfloat16))
        out = torch.zeros(256, 384, device="cuda", dtype=torch.bfloat16)

        def run(st):
            o.gemm_tc(x, w, out, st, pair=kernel == "gemm_tc_pair")

        def check():
            close(out, x.double() @ w.double().t(), "bfloat16")
    else:
        hq, hkv, d, page_size = 4, 2, 128, 16
        decode = kernel.startswith("attn_decode_tma")
        if kernel == "attn_decode_tma_many":  # more blocks than three per SM: the kernel's form for four per SM
            kv_lens, q_lens = [40 + i % 30 for i in range(130)], [1] * 130
        else:
            kv_lens, q_lens = ([300, 200], [1, 1]) if decode else ([300], [300])
        q, k_list, v_list, tables, num_pages = attention_case("bfloat16", hq, hkv, d, page_size, kv_lens, q_lens, None)
        k_pages = dev(paged(k_list, page_size, tables, num_pages, torch.bfloat16))
        v_pages = dev(paged(v_list, page_size, tables, num_pages, torch.bfloat16))
        qd = dev(q)
        out = torch.zeros_like(qd)
        q_start = dev(torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32))
        kv = dev(torch.tensor(kv_lens, dtype=torch.int32))
        table = dev(table_tensor(tables))
        partial = torch.empty(o.decode_partial_numel(len(q_lens), hq, d), device="cuda")

        def run(st):
            if decode:
                o.attn_decode(qd, k_pages, v_pages, out, partial, q_start, kv, table, len(q_lens), d ** -0.5, 0, 2, st,
                              loader="tma")
            else:
                o.attn_tc(qd, k_pages, v_pages, out, q_start, kv, table, 1, q_lens[0], d ** -0.5, st)

        def check():
            want = reference_attention(q.double(), [k.double() for k in k_list], [v.double() for v in v_list], q_lens, None)
            close(out, want, "bfloat16")

    st = status()
    run(st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    check()
    try:
        o.set_wait_test(limit=1 << 14, drop_copy=1)
        run(st)
        torch.cuda.synchronize()
        word = int(st.item())
    finally:
        o.set_wait_test()
    assert word & 16, f"status {word}: the time-out bit is not set"
    assert "wait" in o.describe_status(word)
    st.zero_()
    out.zero_()
    run(st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    check()


def test_sample_greedy_ties_and_all_nan():
    logits = torch.zeros(3, 1000)
    logits[0, [400, 17, 900]] = 5.0
    logits[1] = torch.linspace(-1, 1, 1000)
    logits[2] = float("nan")
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    st = status()
    ops().sample(dev(logits), out, st)
    assert out.tolist()[:2] == [17, 999]
    assert int(st.item()) == 8


@pytest.mark.parametrize("vocab", [331, 151936])
def test_sample_matches_the_plain_generator(vocab):
    g = torch.Generator().manual_seed(17)
    R = 6
    logits = torch.randn(R, vocab, generator=g) * 2
    temps = [0.7, 0.0, 1.3, 0.7, 1.0, 0.2]
    top_k = [0, 0, 40, 5, 1, 0]
    keys = [3, 4, 5, 3, 99, 2 ** 40 + 7]
    pos = [10, 11, 12, 11, 0, 40000]
    seed = 1234
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    st = status()
    ops().sample(dev(logits), out, st, temperature=dev(torch.tensor(temps)), top_k=dev(torch.tensor(top_k, dtype=torch.int32)),
                 request_key=dev(torch.tensor(keys, dtype=torch.int64)), position=dev(torch.tensor(pos, dtype=torch.int32)),
                 seed=seed)
    got = out.tolist()
    want = [plain.sample_token(logits[r], temps[r], top_k[r], seed, keys[r], pos[r]) for r in range(R)]
    assert got == want
    assert got[1] == int(logits[1].argmax()) and got[4] == int(logits[4].argmax())  # greedy row, top-1 row
    assert int(st.item()) == 0


def test_sample_top_k_with_many_equal_logits():
    """Top-k where the k-th largest sits among thousands of logits that share their leading bits (more
    candidates than the kernel's list holds: its slow exact path), where it sits among a handful, and
    where k reaches into equal values (all of them stay candidates); twice in a row on the same rows."""
    g = torch.Generator().manual_seed(23)
    V = 50000
    rows = []
    rows.append(torch.full((V,), 1.5) + 1e-4 * torch.rand(V, generator=g))          # all in one bin
    spread = torch.randn(V, generator=g)
    spread[torch.randperm(V, generator=g)[:7]] += 12.0                                # seven far above the rest
    rows.append(spread)
    flat = torch.zeros(V)
    flat[torch.randperm(V, generator=g)[:30]] = 3.0                                   # thirty equal at the top
    rows.append(flat)
    logits = torch.stack(rows)
    temps, top_k, keys, pos, seed = [0.9, 1.1, 0.8], [300, 5, 12], [1, 2, 3], [7, 8, 9], 77
    want = [plain.sample_token(logits[r], temps[r], top_k[r], seed, keys[r], pos[r]) for r in range(3)]
    st = status()
    for _ in range(2):
        out = torch.full((3,), -1, dtype=torch.int32, device="cuda")
        ops().sample(dev(logits), out, st, temperature=dev(torch.tensor(temps)),
                     top_k=dev(torch.tensor(top_k, dtype=torch.int32)),
                     request_key=dev(torch.tensor(keys, dtype=torch.int64)),
                     position=dev(torch.tensor(pos, dtype=torch.int32)), seed=seed)
        assert out.tolist() == want
    assert int(st.item()) == 0


def test_sampling_follows_the_softmax_distribution():
    """Many draws (different positions) from a small distribution: frequencies match softmax(l / T)."""
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5])
    T, n = 0.8, 20000
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    st = status()
    ops().sample(dev(logits.repeat(n, 1)), out, st, temperature=dev(torch.full((n,), T)),
                 request_key=dev(torch.zeros(n, dtype=torch.int64)),
                 position=dev(torch.arange(n, dtype=torch.int32)), seed=5)
    freq = torch.bincount(out.cpu().long(), minlength=5).double() / n
    want = torch.softmax(logits.double() / T, 0)
    assert float((freq - want).abs().max()) < 0.015  # ~4 standard errors at n = 20000
