"""rms_norm, row reductions and SiLU * Mul on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

# warp-per-row kernel (aligned, <= 1024 f32), CTA-per-row kernel (<= 8192 f32), scalar kernel (odd widths, wider rows)
SHAPES = [(1, 4), (3, 1), (7, 5), (64, 128), (130, 1024), (33, 4096), (9, 8192), (1000, 1000), (129, 516), (5, 12000),
          (2, 70001), (2048, 4096)]


def run_rms_norm(dev, x_host, dtype, eps):
    xd = util.dev_tensor(torch, x_host)
    yd = torch.empty_like(xd)
    dev.rms_norm(dtype, x_host.shape[0], x_host.shape[1], eps, xd.data_ptr(), yd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    return yd.cpu().numpy()


def run_reduce(dev, x_host, dtype, kind):
    xd = util.dev_tensor(torch, x_host)
    yd = torch.empty(x_host.shape[0], dtype=xd.dtype, device="cuda:0")
    dev.reduce(dtype, kind, x_host.shape[0], x_host.shape[1], xd.data_ptr(), yd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    return yd.cpu().numpy()


def run_silu_mul(dev, gate, up, dtype):
    gd = util.dev_tensor(torch, gate)
    ud = None if up is None else util.dev_tensor(torch, up)
    yd = torch.empty_like(gd)
    dev.silu_mul(dtype, gate.shape[0], gate.shape[1], gd.data_ptr(), None if ud is None else ud.data_ptr(), yd.data_ptr(),
                 stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    return yd.cpu().numpy()


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_rms_norm_f32_matches_oracle(dev, pkg, oracle, rows, cols):
    x = util.gen_normal(pkg.capi, (rows, cols), 601, 3.0)
    y = run_rms_norm(dev, x, pkg.capi.F32, 1e-5)
    for ref in (oracle.rms_norm_f32(x, 1e-5), oracle.rms_norm_f32(x, 1e-5, f64_acc=True)):
        m = oracle.compare(y, ref)
        assert m["rel_max"] <= util.F32_REL and m["rel_fro"] <= util.F32_REL, m


@pytest.mark.parametrize("rows,cols", [(1, 8), (33, 4096), (9, 16384), (6, 20000), (5, 333), (512, 4096)])
def test_rms_norm_bf16_matches_oracle(dev, pkg, oracle, rows, cols):
    xb = util.to_bf16(pkg.capi, util.gen_normal(pkg.capi, (rows, cols), 601, 3.0))
    y = run_rms_norm(dev, xb, pkg.capi.BF16, 1e-5).view(np.uint16)
    ref32, ref16 = oracle.rms_norm_bf16(xb, 1e-5)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(y), ref32)
    # the f32 arithmetic before the rounding agrees to ~1e-5 (the bridge sums in index order, the kernel in a
    # tree, and the difference grows with the row length): few outputs may land on the neighbouring bf16 value
    assert np.count_nonzero(y != ref16) <= max(2, y.size // 100)
    assert np.abs(y.astype(np.int32) - ref16.astype(np.int32)).max() <= 1


@pytest.mark.parametrize("rows,cols", SHAPES + [(4, 0)])
def test_reduce_f32_matches_oracle(dev, pkg, oracle, rows, cols):
    x = util.gen_normal(pkg.capi, (rows, cols), 611, 3.0)
    got_max = run_reduce(dev, x, pkg.capi.F32, pkg.capi.REDUCE_MAX)
    assert np.array_equal(got_max, oracle.reduce_f32(x, "max"))  # a maximum is exact
    got_sum = run_reduce(dev, x, pkg.capi.F32, pkg.capi.REDUCE_SUM)
    truth = oracle.reduce_f32(x, "sum", f64_acc=True)
    # sums cancel: the error is measured against the size of the terms, |x|_1 per row
    scale = max(float(np.abs(x).sum(axis=1).max()) if cols else 0.0, 1e-30)
    assert np.abs(got_sum - truth).max() / scale <= util.F32_REL
    # a positive matrix has no cancellation: plain relative error against both oracle variants
    xp = np.abs(x) + 1.0
    got = run_reduce(dev, xp, pkg.capi.F32, pkg.capi.REDUCE_SUM)
    if cols:
        assert np.abs(got / oracle.reduce_f32(xp, "sum", f64_acc=True) - 1).max() <= util.F32_REL
        assert np.abs(got / oracle.reduce_f32(xp, "sum") - 1).max() <= 5 * util.F32_REL  # index-order f32 sum of the bridge


def test_reduce_bf16(dev, pkg, oracle):
    xb = util.to_bf16(pkg.capi, np.abs(util.gen_normal(pkg.capi, (40, 4096), 612)) + 0.5)
    xf = oracle.bf16_to_f32(xb)
    got = oracle.bf16_to_f32(run_reduce(dev, xb, pkg.capi.BF16, pkg.capi.REDUCE_SUM).view(np.uint16))
    assert np.abs(got / oracle.reduce_f32(xf, "sum", f64_acc=True) - 1).max() <= 2.0 ** -8  # one bf16 rounding
    got = oracle.bf16_to_f32(run_reduce(dev, xb, pkg.capi.BF16, pkg.capi.REDUCE_MAX).view(np.uint16))
    assert np.array_equal(got, oracle.reduce_f32(xf, "max"))


@pytest.mark.parametrize("rows,cols", [(1, 4), (7, 5), (64, 128), (33, 4096), (1000, 1001), (2048, 4096)])
@pytest.mark.parametrize("with_up", [True, False])
def test_silu_mul_f32_matches_oracle(dev, pkg, oracle, rows, cols, with_up):
    gate = util.gen_normal(pkg.capi, (rows, cols), 602, 4.0)
    up = util.gen_normal(pkg.capi, (rows, cols), 603) if with_up else None
    y = run_silu_mul(dev, gate, up, pkg.capi.F32)
    for ref in (oracle.silu_mul_f32(gate, up), oracle.silu_mul_f32(gate, up, f64_acc=True)):
        m = oracle.compare(y, ref)
        assert m["rel_max"] <= util.F32_REL and m["rel_fro"] <= util.F32_REL, m
        big = np.abs(ref) >= 1e-30
        assert np.abs(y[big] / ref[big] - 1).max() <= util.F32_REL


def test_silu_mul_bf16_and_f16(dev, pkg, oracle):
    gb = util.to_bf16(pkg.capi, util.gen_normal(pkg.capi, (65, 4096), 602, 4.0))
    ub = util.to_bf16(pkg.capi, util.gen_normal(pkg.capi, (65, 4096), 603))
    y = run_silu_mul(dev, gb, ub, pkg.capi.BF16).view(np.uint16)
    ref32, ref16 = oracle.silu_mul_bf16(gb, ub)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(y), ref32)
    assert np.abs(y.astype(np.int32) - ref16.astype(np.int32)).max() <= 1
    gh = util.f32_to_f16_bits(util.gen_normal(pkg.capi, (9, 1000), 602, 4.0))
    yh = run_silu_mul(dev, gh, None, pkg.capi.F16).view(np.float16).astype(np.float32)
    ref = oracle.silu_mul_f32(gh.view(np.float16).astype(np.float32), None)
    assert np.abs(yh - ref).max() <= 2.0 ** -10 * max(1.0, float(np.abs(ref).max()))


def test_row_operators_reject_bad_arguments(dev, pkg):
    capi = pkg.capi
    with pytest.raises(pkg.hal.HalError):
        dev.rms_norm(capi.F32, 4, 4, 1e-5, 0, 0)
    with pytest.raises(pkg.hal.HalError):
        dev.reduce(capi.F32, 7, 4, 4, 16, 16)
    with pytest.raises(pkg.hal.HalError):
        dev.silu_mul(99, 4, 4, 16, None, 16)


def test_row_operators_full_size_properties(dev, pkg, oracle):
    """65536 x 4096 f32: sampled rows against the oracle plus size-independent properties."""
    capi = pkg.capi
    rows, cols = 65536, 4096
    x = torch.empty(rows, cols, device="cuda:0")
    x.normal_(0.0, 3.0, generator=torch.Generator(device="cuda:0").manual_seed(7))
    y = torch.empty_like(x)
    s = util.cur_stream(torch)
    dev.rms_norm(capi.F32, rows, cols, 0.0, x.data_ptr(), y.data_ptr(), stream=s)
    torch.cuda.synchronize()
    # with eps = 0 every output row has mean square one
    assert float(((y.double() ** 2).mean(dim=1) - 1).abs().max()) <= 1e-5
    idx = torch.tensor([0, 1, 777, 32768, 65535], device="cuda:0")
    ref = oracle.rms_norm_f32(x[idx].cpu().numpy(), 0.0, f64_acc=True)
    assert oracle.compare(y[idx].cpu().numpy(), ref)["rel_max"] <= util.F32_REL
    r = torch.empty(rows, device="cuda:0")
    dev.reduce(capi.F32, capi.REDUCE_MAX, rows, cols, x.data_ptr(), r.data_ptr(), stream=s)
    torch.cuda.synchronize()
    assert torch.equal(r, x.max(dim=1).values)
    dev.reduce(capi.F32, capi.REDUCE_SUM, rows, cols, x.data_ptr(), r.data_ptr(), stream=s)
    torch.cuda.synchronize()
    assert float((r.double() - x.double().sum(dim=1)).abs().max()) <= 1e-5 * float(x.abs().double().sum(dim=1).max())
    dev.silu_mul(capi.F32, rows, cols, x.data_ptr(), None, y.data_ptr(), stream=s)
    torch.cuda.synchronize()
    ref = oracle.silu_mul_f32(x[idx].cpu().numpy(), None, f64_acc=True)
    assert oracle.compare(y[idx].cpu().numpy(), ref)["rel_max"] <= util.F32_REL
    assert dev.status() == 0
