"""Row softmax on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def run_softmax(dev, capi, x_host, dtype):
    xd = util.dev_tensor(torch, x_host)
    yd = torch.empty_like(xd)
    dev.softmax(dtype, x_host.shape[0], x_host.shape[1], xd.data_ptr(), yd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    return yd.cpu().numpy()


# warp kernel (aligned, <= 4096), block kernel (aligned, wider), stream kernel (odd widths / huge rows)
F32_SHAPES = [(1, 4), (3, 1), (7, 5), (64, 128), (33, 4096), (1000, 1000), (129, 516), (5, 12000), (4, 50000),
              (2, 70001), (2048, 4096)]


@pytest.mark.parametrize("rows,cols", F32_SHAPES)
def test_softmax_f32_matches_oracle(dev, pkg, oracle, rows, cols):
    x = util.softmax_input(pkg.capi, rows, cols)
    y = run_softmax(dev, pkg.capi, x, pkg.capi.F32)
    ref = oracle.softmax_f32(x)
    truth = oracle.softmax_f32(x, f64_acc=True)
    for r in (ref, truth):
        m = oracle.compare(y, r, floor_r=1e-30)
        assert m["rel_max"] <= util.F32_REL, m
        assert m["rel_fro"] <= util.F32_REL, m
        assert m["max_elem_rel"] <= util.F32_REL, m  # element-wise, all outputs are positive
    assert np.abs(y.sum(axis=1) - 1.0).max() <= 1e-5


@pytest.mark.parametrize("rows,cols", [(1, 8), (33, 4096), (9, 8192), (6, 20000), (5, 333), (512, 4096)])
def test_softmax_bf16_matches_oracle(dev, pkg, oracle, rows, cols):
    xb = util.to_bf16(pkg.capi, util.softmax_input(pkg.capi, rows, cols))
    y = run_softmax(dev, pkg.capi, xb, pkg.capi.BF16).view(np.uint16)
    ref32, ref16 = oracle.softmax_bf16(xb)
    got = oracle.bf16_to_f32(y)
    m = oracle.compare(got, ref32)
    # one bf16 rounding of a value in [0, 1]: half an ulp is 2^-9 relative
    assert m["max_abs"] <= 2.0 ** -9, m
    assert m["rel_fro"] <= 2.0 ** -8, m
    # the f32 arithmetic before the rounding agrees to 1e-5, so at most a sliver of
    # the outputs may round to the neighbouring bf16 value
    differing = np.count_nonzero(y != ref16)
    assert differing <= max(2, y.size // 1000), differing
    ulp_diff = np.abs(y.astype(np.int32) - ref16.astype(np.int32)).max()
    assert ulp_diff <= 1


def test_softmax_f16(dev, pkg, oracle):
    x = util.softmax_input(pkg.capi, 17, 1024)
    xh = util.f32_to_f16_bits(np.clip(x, -60000, 60000))
    y = run_softmax(dev, pkg.capi, xh, pkg.capi.F16).view(np.float16).astype(np.float32)
    ref = oracle.softmax_f32(xh.view(np.float16).astype(np.float32))
    assert np.abs(y - ref).max() <= 2.0 ** -11 + 1e-7


def test_softmax_empty_and_bad_args(dev, pkg):
    capi = pkg.capi
    x = torch.zeros(16, device="cuda:0")
    dev.softmax(capi.F32, 0, 16, x.data_ptr(), x.data_ptr())  # empty: no-op
    dev.softmax(capi.F32, 4, 0, x.data_ptr(), x.data_ptr())
    with pytest.raises(pkg.hal.KernelError):
        dev.softmax(capi.F32, -1, 16, x.data_ptr(), x.data_ptr())
    with pytest.raises(pkg.hal.KernelError):
        dev.softmax(7, 1, 16, x.data_ptr(), x.data_ptr())
    with pytest.raises(pkg.hal.KernelError):
        dev.softmax(capi.F32, 1, 16, 0, x.data_ptr())


def test_softmax_properties_full_size(dev, pkg, oracle):
    """65536 x 4096 f32: rows sum to one, outliers dominate, sampled rows match the oracle."""
    rows, cols = 65536, 4096
    x = util.softmax_input(pkg.capi, rows, cols)
    xd = util.dev_tensor(torch, x)
    yd = torch.empty_like(xd)
    dev.softmax(pkg.capi.F32, rows, cols, xd.data_ptr(), yd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    sums = yd.sum(dim=1)
    assert float((sums - 1).abs().max()) <= 1e-5
    assert bool((yd >= 0).all())
    # shift invariance: softmax(x + c) == softmax(x)
    y2 = torch.empty_like(xd)
    x2 = xd[:4096] + 1.0
    dev.softmax(pkg.capi.F32, 4096, cols, x2.data_ptr(), y2.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert float((y2[:4096] - yd[:4096]).abs().max()) <= 2e-6
    pick = np.arange(0, rows, 1021)
    y = yd[torch.from_numpy(pick).to("cuda:0")].cpu().numpy()
    m = oracle.compare(y, oracle.softmax_f32(x[pick]), floor_r=1e-30)
    assert m["rel_max"] <= util.F32_REL and m["max_elem_rel"] <= util.F32_REL, m


def test_softmax_host_path(dev, pkg, oracle):
    """Host buffers in, host buffers out (chunked upload / kernel / download)."""
    rows, cols = 6000, 4096  # several 32 MiB chunks
    x = util.softmax_input(pkg.capi, rows, cols, seed=77)
    y = np.empty_like(x)
    dev.softmax_host(pkg.capi.F32, rows, cols, x.ctypes.data, y.ctypes.data)
    m = oracle.compare(y, oracle.softmax_f32(x), floor_r=1e-30)
    assert m["rel_max"] <= util.F32_REL and m["max_elem_rel"] <= util.F32_REL, m
