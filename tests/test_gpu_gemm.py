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
                                       (1024, 1024, 1024, False), (70, 2, 128, True), (3, 1000, 36, False)])
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
