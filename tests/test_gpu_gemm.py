"""GEMM on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def run_gemm(dev, capi, a, b, m, n, k, dtype, out_dtype=None, b_transposed=False, batch=1):
    ad, bd = util.dev_tensor(torch, a), util.dev_tensor(torch, b)
    od = out_dtype if out_dtype is not None else dtype
    tdt = torch.float32 if od == capi.F32 else torch.int16
    # fill with a sentinel so unwritten elements are caught
    cd = torch.full((batch, m, n), 12345 if tdt == torch.int16 else float("nan"), dtype=tdt, device="cuda:0")
    dev.gemm(dtype, m, n, k, ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), out_dtype=out_dtype,
             b_transposed=b_transposed, batch=batch, stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    return cd.cpu().numpy()


# aligned rows (K % 4 == 0, N % 4 == 0): tensor cores with three TF32 products per product, with and without a
# cluster splitting K; anything else: the FP32 pipe
@pytest.mark.parametrize("m,n,k,bt", [(512, 512, 512, False), (512, 512, 512, True), (65, 33, 17, False),
                                       (1, 1, 1, False), (100, 300, 77, True), (130, 70, 260, False),
                                       (100, 300, 76, True), (130, 72, 260, False), (64, 64, 4096, False), (1, 4, 8, False),
                                       (1024, 1024, 1024, False), (70, 2, 128, True), (3, 1000, 36, False),
                                       # more small and ragged shapes of the warp-level kernel
                                       (384, 640, 512, False), (384, 640, 512, True), (128, 128, 64, False), (129, 132, 68, True),
                                       (1200, 1400, 128, False), (256, 256, 2048, False), (200, 12, 300, False)])
def test_gemm_f32(dev, pkg, oracle, m, n, k, bt):
    capi = pkg.capi
    a = util.gen_uniform(capi, (m, k), 101)
    b = util.gen_uniform(capi, (n, k) if bt else (k, n), 102)
    c = run_gemm(dev, capi, a, b, m, n, k, capi.F32, b_transposed=bt)[0]
    for ref in (oracle.gemm_f32(a, b, bt), oracle.gemm_f32(a, b, bt, f64_acc=True)):
        mt = oracle.compare(c, ref)
        assert mt["rel_max"] <= util.F32_REL, mt
        assert mt["rel_fro"] <= util.F32_REL, mt


def test_gemm_f32_wide_dynamic_range_and_batch(dev, pkg, oracle):
    """Entries spread over six decades: the split into hi and lo halves must keep f32 accuracy for every magnitude."""
    capi = pkg.capi
    batch, m, n, k = 3, 96, 80, 512
    mag = 10.0 ** (3.0 * util.gen_uniform(capi, (batch, m, k), 111))
    a = (util.gen_uniform(capi, (batch, m, k), 112) * mag).astype(np.float32)
    b = util.gen_normal(capi, (batch, k, n), 113)
    c = run_gemm(dev, capi, a, b, m, n, k, capi.F32, batch=batch)
    for i in range(batch):
        truth = oracle.gemm_f32(a[i], b[i], False, f64_acc=True)
        # row-wise bound: every output row against the largest magnitude of that row (rows differ by decades)
        err = np.abs(c[i] - truth).max(axis=1) / np.abs(truth).max(axis=1)
        assert err.max() <= util.F32_REL, err.max()


TC_SHAPES = [
    (128, 256, 64, False), (128, 256, 64, True),        # one tile, one k-block
    (128, 256, 256, False), (128, 256, 256, True),      # one tile, ring wraps
    (256, 512, 512, False), (256, 512, 512, True),      # several tiles
    (200, 264, 136, False), (200, 264, 136, True),      # ragged M, N, K (multiples of 8)
    (1024, 1024, 1024, False), (4096, 512, 384, True),
]


@pytest.mark.parametrize("m,n,k,bt", TC_SHAPES)
def test_gemm_bf16_tensor_core(dev, pkg, oracle, m, n, k, bt):
    capi = pkg.capi
    sigma = k ** -0.25
    a = util.to_bf16(capi, util.gen_normal(capi, (m, k), 301, sigma))
    b = util.to_bf16(capi, util.gen_normal(capi, (n, k) if bt else (k, n), 302, sigma))
    c = run_gemm(dev, capi, a, b, m, n, k, capi.BF16, b_transposed=bt)[0].view(np.uint16)
    ref32, ref16 = oracle.gemm_bf16(a, b, bt)
    got = oracle.bf16_to_f32(c)
    util.assert_16bit_close(oracle, got, ref32)
    # the rounded results agree with the oracle's own rounding except where the f32 sums
    # (accumulated in a different order) straddle a rounding boundary
    assert np.count_nonzero(c != ref16) <= c.size // 50


def test_gemm_bf16_f32_out_and_batch(dev, pkg, oracle):
    capi = pkg.capi
    batch, m, n, k = 3, 256, 256, 192
    a = util.to_bf16(capi, util.gen_normal(capi, (batch, m, k), 310, 0.3))
    b = util.to_bf16(capi, util.gen_normal(capi, (batch, k, n), 311, 0.3))
    c = run_gemm(dev, capi, a, b, m, n, k, capi.BF16, out_dtype=capi.F32, batch=batch)
    for i in range(batch):
        ref32, _ = oracle.gemm_bf16(a[i], b[i])
        mt = oracle.compare(c[i], ref32)
        assert mt["rel_max"] <= 1e-5 and mt["rel_fro"] <= 1e-5, (i, mt)  # f32 accumulate, f32 out


def test_gemm_f16_tensor_core(dev, pkg, oracle):
    capi = pkg.capi
    m, n, k = 256, 256, 128
    a32 = util.gen_normal(capi, (m, k), 320, 0.3)
    b32 = util.gen_normal(capi, (k, n), 321, 0.3)
    a, b = util.f32_to_f16_bits(a32), util.f32_to_f16_bits(b32)
    c = run_gemm(dev, capi, a, b, m, n, k, capi.F16, out_dtype=capi.F32)[0]
    ref = oracle.gemm_f32(a.view(np.float16).astype(np.float32), b.view(np.float16).astype(np.float32))
    mt = oracle.compare(c, ref)
    assert mt["rel_max"] <= 1e-5, mt


def test_gemm_bf16_odd_shape_falls_to_fp32_pipe(dev, pkg, oracle):
    """Leading dimensions that are not 16-byte multiples cannot use TMA; still on the GPU."""
    capi = pkg.capi
    m, n, k = 50, 30, 20
    a = util.to_bf16(capi, util.gen_normal(capi, (m, k), 330, 0.5))
    b = util.to_bf16(capi, util.gen_normal(capi, (k, n), 331, 0.5))
    c = run_gemm(dev, capi, a, b, m, n, k, capi.BF16)[0].view(np.uint16)
    ref32, _ = oracle.gemm_bf16(a, b)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(c), ref32)


def test_gemm_edge_cases(dev, pkg):
    capi = pkg.capi
    t = torch.zeros(64, device="cuda:0")
    p = t.data_ptr()
    dev.gemm(capi.F32, 0, 8, 8, p, p, p)  # empty output
    c = torch.full((4, 4), 7.0, device="cuda:0")
    dev.gemm(capi.F32, 4, 4, 0, p, p, c.data_ptr())  # empty contraction: C = 0
    torch.cuda.synchronize()
    assert float(c.abs().max()) == 0.0
    with pytest.raises(pkg.hal.KernelError):
        dev.gemm(capi.F32, 4, 4, 4, p, p, p, out_dtype=capi.BF16)
    with pytest.raises(pkg.hal.KernelError):
        dev.gemm(capi.F32, -4, 4, 4, p, p, p)


def test_gemm_bf16_full_size_sampled_rows(dev, pkg, oracle):
    """8192^3: sampled output rows against the oracle, plus linearity C(2A) == 2 C(A) exactly."""
    capi = pkg.capi
    n = 8192
    sigma = n ** -0.25
    a = util.to_bf16(capi, util.gen_normal(capi, (n, n), 301, sigma))
    b = util.to_bf16(capi, util.gen_normal(capi, (n, n), 302, sigma))
    ad, bd = util.dev_tensor(torch, a), util.dev_tensor(torch, b)
    cd = torch.empty((n, n), dtype=torch.int16, device="cuda:0")
    dev.gemm(capi.BF16, n, n, n, ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    rows = np.array([0, 1, 127, 128, 4095, 4096, 5000, 8191])
    got = oracle.bf16_to_f32(cd[torch.from_numpy(rows).to("cuda:0")].cpu().numpy().view(np.uint16))
    ref32, _ = oracle.gemm_bf16(np.ascontiguousarray(a[rows]), b)
    util.assert_16bit_close(oracle, got, ref32)
    # scaling A by two is exact in bf16 and in f32 accumulation
    a2 = (ad.view(torch.bfloat16) * 2).view(torch.int16)
    c2 = torch.empty_like(cd)
    dev.gemm(capi.BF16, n, n, n, a2.data_ptr(), bd.data_ptr(), c2.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert torch.equal(c2.view(torch.bfloat16), cd.view(torch.bfloat16) * 2)


def test_gemm_host_path(dev, pkg, oracle):
    capi = pkg.capi
    m, n, k = 2304, 512, 4096  # several A row blocks
    a = util.to_bf16(capi, util.gen_normal(capi, (m, k), 340, k ** -0.25))
    b = util.to_bf16(capi, util.gen_normal(capi, (k, n), 341, k ** -0.25))
    c = np.zeros((m, n), np.uint16)
    dev.gemm_host(capi.BF16, m, n, k, a.ctypes.data, b.ctypes.data, c.ctypes.data)
    ref32, _ = oracle.gemm_bf16(a, b)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(c), ref32)


@pytest.mark.parametrize("dtype,m,n,k,n0,nb,bt", [
    ("bf16", 512, 1024, 256, 256, 512, False),   # CTA-pair kernel on a column block of a wider matrix
    ("bf16", 512, 1024, 256, 512, 256, True),    # B stored [N, K]: the block is a row range of it, C still pitched
    ("bf16", 96, 768, 128, 256, 256, False),     # single-CTA tensor-core kernel
    ("bf16", 50, 60, 20, 10, 30, False),         # FP32-pipe kernel (pitches not 16-byte multiples)
    ("f32", 256, 768, 128, 256, 256, False),     # three-TF32 kernel
    ("f32", 64, 512, 2048, 128, 64, True),       # the same with a cluster splitting K
    ("f32", 33, 50, 17, 7, 21, False),           # FP32 pipe
])
def test_gemm_column_block_in_place(dev, pkg, oracle, dtype, m, n, k, n0, nb, bt):
    """C[:, n0:n0+nb] = A * B[:, n0:n0+nb] with B and C addressed inside their full row-major matrices through
    ldb / ldc (the N-column split of one large GEMM); every other column of C keeps its sentinel."""
    capi = pkg.capi
    sigma = k ** -0.25
    a32 = util.gen_normal(capi, (m, k), 350, sigma)
    b32 = util.gen_normal(capi, (n, k) if bt else (k, n), 351, sigma)
    if dtype == "bf16":
        a, b, code, tdt, es = util.to_bf16(capi, a32), util.to_bf16(capi, b32), capi.BF16, torch.int16, 2
    else:
        a, b, code, tdt, es = a32, b32, capi.F32, torch.float32, 4
    ad, bd = util.dev_tensor(torch, a), util.dev_tensor(torch, b)
    sentinel = 12345 if tdt == torch.int16 else 777.0
    cd = torch.full((m, n), sentinel, dtype=tdt, device="cuda:0")
    b_ptr = bd.data_ptr() + (n0 * k * es if bt else n0 * es)  # rows n0.. of [N, K], or columns n0.. of [K, N]
    dev.gemm(code, m, nb, k, ad.data_ptr(), b_ptr, cd.data_ptr() + n0 * es, b_transposed=bt,
             ldb=(k if bt else n), ldc=n, stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    c = cd.cpu().numpy()
    blk = np.ascontiguousarray(b[n0:n0 + nb] if bt else b[:, n0:n0 + nb])
    if dtype == "bf16":
        ref32, _ = oracle.gemm_bf16(a, blk, b_transposed=bt)
        util.assert_16bit_close(oracle, oracle.bf16_to_f32(np.ascontiguousarray(c[:, n0:n0 + nb]).view(np.uint16)), ref32)
    else:
        mt = oracle.compare(np.ascontiguousarray(c[:, n0:n0 + nb]), oracle.gemm_f32(a, blk, b_transposed=bt, f64_acc=True))
        assert mt["rel_max"] <= util.F32_REL and mt["rel_fro"] <= util.F32_REL, mt
    outside = np.concatenate([c[:, :n0].ravel(), c[:, n0 + nb:].ravel()])
    assert (outside == sentinel).all()
    with pytest.raises(pkg.hal.KernelError, match="pitch"):
        dev.gemm(code, m, nb, k, ad.data_ptr(), b_ptr, cd.data_ptr(), ldc=nb - 1)


def test_gemm_host_pitched(dev, pkg, oracle):
    """tsm100_gemm_host on a column block of host matrices (what the launcher's N-column split does per device)."""
    capi = pkg.capi
    m, n, k, n0, nb = 640, 1024, 512, 512, 256
    a = util.to_bf16(capi, util.gen_normal(capi, (m, k), 360, k ** -0.25))
    b = util.to_bf16(capi, util.gen_normal(capi, (k, n), 361, k ** -0.25))
    c = np.full((m, n), 12345, np.uint16)
    dev.gemm_host(capi.BF16, m, nb, k, a.ctypes.data, b.ctypes.data + n0 * 2, c.ctypes.data + n0 * 2, ldb=n, ldc=n)
    ref32, _ = oracle.gemm_bf16(a, np.ascontiguousarray(b[:, n0:n0 + nb]))
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(np.ascontiguousarray(c[:, n0:n0 + nb])), ref32)
    assert (c[:, :n0] == 12345).all() and (c[:, n0 + nb:] == 12345).all()


def test_gemm_bf16_batched_64x4096_strides(dev, pkg, oracle):
    """The batched configuration at full size (64 problems of 4096^3, 6 GiB): problem i is problem 0 with A scaled by
    2^(i-32) and B by 2^((7i mod 64)-32) - exact in bf16 and in the f32 accumulation - so C_i must equal
    2^(a_i+b_i) * C_0 bit for bit; reading or writing any problem at a wrong batch offset breaks that.
    Problem 0 itself is checked against the oracle on sampled rows."""
    capi = pkg.capi
    n, batch = 4096, 64
    sigma = n ** -0.25
    a0 = util.to_bf16(capi, util.gen_normal(capi, (n, n), 310, sigma))
    b0 = util.to_bf16(capi, util.gen_normal(capi, (n, n), 311, sigma))
    a0d, b0d = util.dev_tensor(torch, a0).view(torch.bfloat16), util.dev_tensor(torch, b0).view(torch.bfloat16)
    ea = torch.arange(batch, device="cuda:0") - 32
    eb = (torch.arange(batch, device="cuda:0") * 7) % 64 - 32
    ad = (a0d[None] * torch.pow(2.0, ea.float())[:, None, None].to(torch.bfloat16)).contiguous()
    bd = (b0d[None] * torch.pow(2.0, eb.float())[:, None, None].to(torch.bfloat16)).contiguous()
    cd = torch.empty((batch, n, n), dtype=torch.bfloat16, device="cuda:0")
    dev.gemm(capi.BF16, n, n, n, ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), batch=batch, stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    i0 = int(torch.nonzero((ea + eb) == 0)[0])  # a problem whose scales cancel: C_i0 == C_unscaled
    base = cd[i0].float()
    for i in range(batch):
        assert torch.equal(cd[i].float(), base * float(2.0 ** int(ea[i] + eb[i]))), i
    rows = np.array([0, 129, 2047, 4095])
    got = oracle.bf16_to_f32(cd[i0].view(torch.int16)[torch.from_numpy(rows).to("cuda:0")].cpu().numpy().view(np.uint16))
    ref32, _ = oracle.gemm_bf16(np.ascontiguousarray(a0[rows]), b0)
    util.assert_16bit_close(oracle, got, ref32, "64 x 4096^3, problem with unit scale", report=True)


@pytest.mark.parametrize("m,n,k,bt,batch", [
    (2048, 2048, 2048, False, 1), (1024, 4096, 4096, True, 1), (1032, 2052, 1028, False, 1), (1100, 2100, 300, True, 1),
    (1024, 2048, 512, False, 3), (4096, 4096, 4096, False, 1), (2048, 2048, 8192, False, 1),
    (128, 16640, 512, False, 1), (100, 16384, 260, True, 1)])  # one row block: the single-CTA form of the kernel
def test_gemm_f32_tcgen05(dev, pkg, oracle, m, n, k, bt, batch):
    """Large f32 problems run on the tcgen05 kernel (hi / lo planes, three TF32 products, chunked accumulation):
    sampled rows against the float64-accumulating oracle at the 1e-5 bar, ragged edges and batches included, and
    against the f32-accumulating oracle's own distance from float64 for context."""
    capi = pkg.capi
    a = util.gen_uniform(capi, (batch, m, k), 101)
    b = util.gen_uniform(capi, (batch, n, k) if bt else (batch, k, n), 102)
    c = run_gemm(dev, capi, a, b, m, n, k, capi.F32, b_transposed=bt, batch=batch)
    assert not np.isnan(c).any()
    rows = np.array(sorted({r for r in (0, 1, 127, 128, m // 2 + 3, m - 1) if r < m}))
    for i in range(batch):
        ref = oracle.gemm_f32(np.ascontiguousarray(a[i][rows]), b[i], b_transposed=bt, f64_acc=True)
        mt = oracle.compare(np.ascontiguousarray(c[i][rows]), ref)
        f32 = oracle.compare(oracle.gemm_f32(np.ascontiguousarray(a[i][rows]), b[i], b_transposed=bt), ref)
        print(f"[parity] f32 GEMM {m}x{n}x{k} problem {i}: GPU rel_max {mt['rel_max']:.2e} rel_fro {mt['rel_fro']:.2e}; "
              f"f32 CPU loop rel_max {f32['rel_max']:.2e} rel_fro {f32['rel_fro']:.2e}")
        assert mt["rel_max"] <= util.F32_REL and mt["rel_fro"] <= util.F32_REL, (i, mt)


@pytest.mark.parametrize("bt", [False, True])
def test_gemm_bf16_batch_members_give_equal_bits_and_row_blocks_agree(dev, pkg, bt):
    """The pair kernel walks K backwards in every other wave of tiles, counted inside a tile's own problem: equal
    problems give equal bits wherever they stand in a batch and when launched alone.  A row block of a problem
    launched on its own (what the host-buffer call streams) has other waves, so its f32 sums are taken in another
    order: it agrees with the whole problem to one rounding of the 16-bit result."""
    capi = pkg.capi
    m, n, k = 4352, 4096, 2048   # 17 row tiles: a full band of 16 and a band of one
    g = torch.Generator(device="cuda:0").manual_seed(77)
    a = (torch.randn(m, k, device="cuda:0", generator=g) * k ** -0.25).to(torch.bfloat16)
    b = (torch.randn((n, k) if bt else (k, n), device="cuda:0", generator=g) * k ** -0.25).to(torch.bfloat16)
    whole = torch.empty(m, n, dtype=torch.bfloat16, device="cuda:0")
    st = util.cur_stream(torch)
    dev.gemm(capi.BF16, m, n, k, a.data_ptr(), b.data_ptr(), whole.data_ptr(), b_transposed=bt, stream=st)
    for r0, rows in ((0, 1024), (1024, 256), (1280, 3072)):
        part = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda:0")
        dev.gemm(capi.BF16, rows, n, k, a[r0:].data_ptr(), b.data_ptr(), part.data_ptr(), b_transposed=bt, stream=st)
        torch.cuda.synchronize()
        x, y = part.float(), whole[r0:r0 + rows].float()
        # one bf16 step at that magnitude, at most; results near zero (cancelling sums of O(1) terms) differ by the f32 sums' own error
        ulp = torch.maximum(x.abs(), y.abs()) * 2.0 ** -7 + 1e-5
        assert bool(((x - y).abs() <= ulp).all()), (r0, rows)
        assert float((x != y).float().mean()) <= 0.02, (r0, rows)
    # the same problem twice in a batch of three beside a different one, and alone
    a3 = torch.stack([a[:1024], a[1024:2048], a[:1024]]).contiguous()
    b3 = b[None].expand(3, *b.shape).contiguous()
    c3 = torch.empty(3, 1024, n, dtype=torch.bfloat16, device="cuda:0")
    dev.gemm(capi.BF16, 1024, n, k, a3.data_ptr(), b3.data_ptr(), c3.data_ptr(), b_transposed=bt, batch=3, stream=st)
    alone = torch.empty(1024, n, dtype=torch.bfloat16, device="cuda:0")
    dev.gemm(capi.BF16, 1024, n, k, a.data_ptr(), b.data_ptr(), alone.data_ptr(), b_transposed=bt, stream=st)
    torch.cuda.synchronize()
    assert dev.status() == 0
    assert torch.equal(c3[0].view(torch.int16), c3[2].view(torch.int16))
    assert torch.equal(c3[0].view(torch.int16), alone.view(torch.int16))
