"""The multi-GPU launcher's host logic on a machine without GPUs: how a problem is dealt out
(tsm100_multi_plan), and how tsm100_multi_run_with schedules, watches and reports per-device
workers - here Python stand-ins for devices, some of which fail, raise or overrun their limit.
Nothing in this file touches a GPU."""
import time

import numpy as np
import pytest


def _softmax_rows(x):
    e = np.exp(x - x.max(axis=1, keepdims=True))
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


def test_plan_tiles_every_problem(pkg):
    L, capi = pkg.launcher, pkg.capi
    # softmax rows, ragged
    job = L.softmax_job(capi.F32, 65537, 4096, 0, 0)
    sh = [job.plan(8, i) for i in range(8)]
    assert sh[0].first == 0 and sh[-1].stop == 65537 and all(a.stop == b.first for a, b in zip(sh, sh[1:]))
    assert {s.count for s in sh} == {8192, 8193} and sh[0].count == 8193
    # one large GEMM: N columns in whole 256-column tiles
    job = L.gemm_job(capi.BF16, 8192, 8192, 8192, 0, 0, 0)
    sh = [job.plan(8, i) for i in range(8)]
    assert [(s.first, s.count) for s in sh] == [(i * 1024, 1024) for i in range(8)]
    job = L.gemm_job(capi.BF16, 64, 1000, 64, 0, 0, 0)
    assert [(s.first, s.count) for s in (job.plan(3, i) for i in range(3))] == [(0, 512), (512, 256), (768, 232)]
    # more devices than tiles: the last ones get nothing
    assert [job.plan(8, i).count for i in range(8)] == [256, 256, 256, 232, 0, 0, 0, 0]
    # batched GEMM: problems; attention: (batch, KV head) groups
    job = L.gemm_job(capi.BF16, 4096, 4096, 4096, 0, 0, 0, batch=64)
    assert [job.plan(8, i).count for i in range(8)] == [8] * 8
    job = L.attention_job(capi.BF16, 2, 64, 8, 16384, 128, 0, 0, 0, 0, causal=True)
    assert [(s.first, s.count) for s in (job.plan(8, i) for i in range(8))] == [(2 * i, 2) for i in range(8)]
    # a pitched batched GEMM cannot be split by problems; bad indices are refused
    with pytest.raises(pkg.hal.HalError, match="packed"):
        L.gemm_job(capi.BF16, 64, 64, 64, 0, 0, 0, batch=2, lda=128).plan(2, 0)
    with pytest.raises(pkg.hal.HalError, match="bad device index"):
        L.softmax_job(capi.F32, 8, 8, 0, 0).plan(2, 2)


def test_fake_devices_compute_their_shards(pkg):
    """Four stand-in devices each do their rows of a softmax on the caller's host buffers."""
    L, capi = pkg.launcher, pkg.capi
    rows, cols = 37, 64
    x = np.random.default_rng(3).standard_normal((rows, cols)).astype(np.float32)
    y = np.zeros_like(x)
    seen = {}

    def worker(job, ordinal, first, count, rep):
        seen[ordinal] = (first, count)
        y[first:first + count] = _softmax_rows(x[first:first + count])
        rep.kernel_ms = 1.5
        return capi.OK

    job = L.softmax_job(capi.F32, rows, cols, x.ctypes.data, y.ctypes.data, launches=3)
    reps = L.MultiGpuLauncher([3, 1, 4, 0]).run(job, worker)
    assert np.array_equal(y, _softmax_rows(x))
    assert [r.ordinal for r in reps] == [3, 1, 4, 0] and all(r.status == capi.OK for r in reps)
    assert [(r.first, r.count) for r in reps] == [(0, 10), (10, 9), (19, 9), (28, 9)]
    assert seen == {3: (0, 10), 1: (10, 9), 4: (19, 9), 0: (28, 9)}
    assert all(abs(r.kernel_ms - 1.5) < 1e-6 and r.total_ms >= 0 for r in reps)


def test_a_failing_device_is_named(pkg):
    L, capi = pkg.launcher, pkg.capi

    def worker(job, ordinal, first, count, rep):
        if ordinal == 5:
            rep.message = b"injected launch failure"
            return capi.ERR_LAUNCH
        return capi.OK

    ml = L.MultiGpuLauncher([2, 5, 7])
    with pytest.raises(pkg.hal.KernelError, match="device 5: injected launch failure"):
        ml.run(L.softmax_job(capi.F32, 30, 8, 0, 0), worker)
    assert [r.status for r in ml.last_reports] == [capi.OK, capi.ERR_LAUNCH, capi.OK]
    assert "device 5" in ml.last_reports[1].message


def test_a_worker_that_raises_is_a_failed_device(pkg):
    L, capi = pkg.launcher, pkg.capi

    def worker(job, ordinal, first, count, rep):
        if ordinal == 1:
            raise ValueError("worker exploded")
        return capi.OK

    ml = L.MultiGpuLauncher([0, 1])
    with pytest.raises(pkg.hal.HalError, match="device 1: worker exploded"):
        ml.run(L.softmax_job(capi.F32, 4, 8, 0, 0), worker)
    assert ml.last_reports[0].status == capi.OK


def test_a_slow_device_runs_into_the_limit(pkg):
    L, capi = pkg.launcher, pkg.capi

    def worker(job, ordinal, first, count, rep):
        if ordinal == 6:
            time.sleep(0.4)  # a stuck device, as far as the launcher can tell
        return capi.OK

    ml = L.MultiGpuLauncher([4, 6])
    t0 = time.perf_counter()
    with pytest.raises(pkg.hal.HalError, match=r"device 6 did not finish within 100 ms"):
        ml.run(L.softmax_job(capi.F32, 4, 8, 0, 0, timeout_ms=100), worker)
    assert time.perf_counter() - t0 >= 0.35  # the call returns only after the late device has drained
    assert [r.status for r in ml.last_reports] == [capi.OK, capi.ERR_TIMEOUT]
    # without a limit the same run is fine
    ml.run(L.softmax_job(capi.F32, 4, 8, 0, 0), worker)


def test_bad_device_lists(pkg):
    L, capi = pkg.launcher, pkg.capi
    with pytest.raises(ValueError):
        L.MultiGpuLauncher([])
    with pytest.raises(pkg.hal.HalError, match="listed twice"):
        L.MultiGpuLauncher([1, 1]).run(L.softmax_job(capi.F32, 4, 8, 0, 0), lambda *a: capi.OK)


def test_builtin_worker_without_a_gpu_reports_the_device(pkg):
    """No CPU fallback: on a machine without a CUDA device the built-in worker fails and says which device."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    L, capi = pkg.launcher, pkg.capi
    x = np.zeros((4, 8), np.float32)
    ml = L.MultiGpuLauncher([0])
    with pytest.raises(pkg.hal.BackendNotAvailable, match="device 0"):
        ml.run(L.softmax_job(capi.F32, 4, 8, x.ctypes.data, x.ctypes.data))
