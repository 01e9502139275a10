"""tsm100_multi_run on real devices: every visible GPU gets its shard of a problem given once on host buffers."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _ordinals(pkg):
    return list(range(pkg.hal.CudaSm100Device.device_count()))


def test_softmax_over_all_devices(pkg, oracle):
    L, capi = pkg.launcher, pkg.capi
    ords = _ordinals(pkg)
    x = util.softmax_input(capi, 4099, 4096)  # ragged over any device count
    y = np.zeros_like(x)
    ml = L.MultiGpuLauncher(ords)
    reps = ml.run(L.softmax_job(capi.F32, 4099, 4096, x.ctypes.data, y.ctypes.data, launches=2, timeout_ms=60000))
    assert sum(r.count for r in reps) == 4099 and all(r.status == 0 and r.device_status == 0 for r in reps)
    assert all(r.kernel_ms > 0 for r in reps if r.count)
    m = oracle.compare(y, oracle.softmax_f32(x, f64_acc=True), floor_r=1e-30)
    assert m["rel_max"] <= util.F32_REL and m["max_elem_rel"] <= util.F32_REL, m


def test_gemm_column_split_in_place(pkg, oracle):
    """One GEMM split by N columns: each device reads its columns of the host's row-major B and writes its columns of C."""
    L, capi = pkg.launcher, pkg.capi
    ords = _ordinals(pkg)
    m, n, k = 512, 2048, 1024
    a = util.to_bf16(capi, util.gen_normal(capi, (m, k), 301, k ** -0.25))
    b = util.to_bf16(capi, util.gen_normal(capi, (k, n), 302, k ** -0.25))
    c = np.full((m, n), 12345, np.uint16)
    ml = L.MultiGpuLauncher(ords)
    reps = ml.run(L.gemm_job(capi.BF16, m, n, k, a.ctypes.data, b.ctypes.data, c.ctypes.data))
    assert [r.first for r in reps][0] == 0 and sum(r.count for r in reps) == n
    ref32, _ = oracle.gemm_bf16(a, b)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(c), ref32)
    # B stored [N, K] and an f32 problem through the same split
    bt = np.ascontiguousarray(b.T)
    c2 = np.zeros((m, n), np.uint16)
    ml.run(L.gemm_job(capi.BF16, m, n, k, a.ctypes.data, bt.ctypes.data, c2.ctypes.data, b_transposed=True))
    assert np.array_equal(c2, c)
    af, bf = util.gen_uniform(capi, (256, 512), 101), util.gen_uniform(capi, (512, 768), 102)
    cf = np.zeros((256, 768), np.float32)
    ml.run(L.gemm_job(capi.F32, 256, 768, 512, af.ctypes.data, bf.ctypes.data, cf.ctypes.data))
    mt = oracle.compare(cf, oracle.gemm_f32(af, bf, f64_acc=True))
    assert mt["rel_max"] <= util.F32_REL and mt["rel_fro"] <= util.F32_REL, mt


def test_batched_gemm_and_attention_groups(pkg, oracle):
    L, capi = pkg.launcher, pkg.capi
    ords = _ordinals(pkg)
    ml = L.MultiGpuLauncher(ords)
    batch, m = 5, 256
    a = util.to_bf16(capi, util.gen_normal(capi, (batch, m, m), 310, 0.3))
    b = util.to_bf16(capi, util.gen_normal(capi, (batch, m, m), 311, 0.3))
    c = np.zeros((batch, m, m), np.uint16)
    ml.run(L.gemm_job(capi.BF16, m, m, m, a.ctypes.data, b.ctypes.data, c.ctypes.data, batch=batch))
    for i in range(batch):
        ref32, _ = oracle.gemm_bf16(a[i], b[i])
        util.assert_16bit_close(oracle, oracle.bf16_to_f32(c[i]), ref32, i)
    q = util.to_bf16(capi, util.gen_normal(capi, (2, 8, 512, 128), 501))
    k = util.to_bf16(capi, util.gen_normal(capi, (2, 2, 512, 128), 502))
    v = util.to_bf16(capi, util.gen_normal(capi, (2, 2, 512, 128), 503))
    o = np.zeros_like(q)
    reps = ml.run(L.attention_job(capi.BF16, 2, 8, 2, 512, 128, q.ctypes.data, k.ctypes.data, v.ctypes.data, o.ctypes.data,
                                  causal=True))
    assert sum(r.count for r in reps) == 4
    ref32, _ = oracle.attention_bf16(q, k, v, True)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)
    L.MultiGpuLauncher.release()


def test_a_missing_device_is_named(pkg):
    L, capi = pkg.launcher, pkg.capi
    x = np.zeros((8, 64), np.float32)
    ml = L.MultiGpuLauncher([0, 57])
    with pytest.raises(pkg.hal.HalError, match="device 57"):
        ml.run(L.softmax_job(capi.F32, 8, 64, x.ctypes.data, x.ctypes.data))
    assert ml.last_reports[0].status == 0 and ml.last_reports[1].status != 0
