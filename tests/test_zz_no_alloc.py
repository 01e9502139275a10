"""The allocation-free GEMM entry point, called through the C ABI.

`tsm100_gemm_static_scratch` serves callers that cannot call cudaMalloc (code running
beside a CUDA-graph capture, hosts with a frozen device heap, loops that cannot take
cudaMalloc's implicit synchronisation): its scratch word sits in a static device array
inside the library.  It must give exactly what `tsm100_gemm` gives, on two calls in a
row (the array is shared and keeps the previous call's contents).  This file sorts
last on purpose, so a failure here cannot hide the other tests in a run that stops at
the first failure.
"""
import ctypes as C

import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _case(capi, m, n, k, seed):
    a = util.to_bf16(capi, util.gen_normal(capi, (m, k), seed, k ** -0.25))
    b = util.to_bf16(capi, util.gen_normal(capi, (k, n), seed + 1, k ** -0.25))
    return util.dev_tensor(torch, a), util.dev_tensor(torch, b)


def test_static_scratch_gemm_matches_gemm_twice(dev, pkg):
    capi, lib = pkg.capi, pkg.capi.lib()
    stream = util.cur_stream(torch)
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    for call, (m, n, k, seed) in enumerate([(384, 512, 320, 901), (256, 264, 1024, 905)]):
        ad, bd = _case(capi, m, n, k, seed)
        want = torch.full((m, n), 12345, dtype=torch.int16, device="cuda:0")
        got = torch.full((m, n), 12345, dtype=torch.int16, device="cuda:0")
        dev.gemm(capi.BF16, m, n, k, ad.data_ptr(), bd.data_ptr(), want.data_ptr(), stream=stream)
        d = capi.GemmDesc(capi.BF16, capi.BF16, 0, 1, m, n, k)
        status[0] = -1
        st = lib.tsm100_gemm_static_scratch(C.byref(d), ad.data_ptr(), bd.data_ptr(), got.data_ptr(), stream or None,
                                            C.cast(status.data_ptr(), C.POINTER(C.c_uint32)))
        assert st == capi.OK, capi.last_error()
        torch.cuda.synchronize()
        assert int(status[0]) == 0, f"call {call}: kernel status {int(status[0]):#x}"
        # same kernel, same inputs: bit-identical (the tolerance of the other GEMM tests is not needed)
        assert torch.equal(got, want), f"call {call}: static-scratch GEMM differs from tsm100_gemm"
        assert int((got == 12345).sum()) < got.numel() // 100
    assert dev.status() == 0


def test_static_scratch_gemm_rejects_what_it_cannot_take(pkg):
    capi, lib = pkg.capi, pkg.capi.lib()
    x = torch.zeros(64 * 64, device="cuda:0")
    p = x.data_ptr()
    for desc, frag in [(capi.GemmDesc(capi.F32, capi.F32, 0, 1, 64, 64, 64), "only the tensor-core kernel"),
                       (capi.GemmDesc(capi.BF16, capi.BF16, 0, 1, 64, 30, 64), "only the tensor-core kernel"),
                       (capi.GemmDesc(capi.BF16, capi.BF16, 0, 1, 0, 64, 64), "must be positive")]:
        assert lib.tsm100_gemm_static_scratch(C.byref(desc), p, p, p, None, None) == capi.ERR_INVALID
        assert frag in capi.last_error(), capi.last_error()
    d = capi.GemmDesc(capi.BF16, capi.BF16, 0, 1, 64, 64, 64)
    assert lib.tsm100_gemm_static_scratch(C.byref(d), None, p, p, None, None) == capi.ERR_INVALID
