"""Helpers for the parity tests: seeded inputs from the library's generator,
torch tensors as device memory, tolerances of the hot-path contract."""
from __future__ import annotations

import ctypes as C

import numpy as np

# Tolerances (f32 GEMM and softmax: relative error <= 1e-5; 16-bit GEMM and
# attention: max-abs <= 2e-2 and relative Frobenius <= 1e-2 against the
# unrounded f32 oracle).
F32_REL = 1e-5
BF16_MAX_ABS = 2e-2
BF16_REL_FRO = 1e-2


def gen_uniform(capi, shape, seed, first=0):
    out = np.empty(shape, np.float32)
    assert capi.lib().tsm100_fill_uniform_f32(out.ctypes.data, out.size, seed, first) == 0
    return out


def gen_normal(capi, shape, seed, sigma=1.0, first=0):
    out = np.empty(shape, np.float32)
    assert capi.lib().tsm100_fill_normal_f32(out.ctypes.data, out.size, seed, first, float(sigma)) == 0
    return out


def plant_outliers(capi, arr, seed, period=100, value=20.0, first=0):
    assert capi.lib().tsm100_plant_outliers_f32(arr.ctypes.data, arr.size, seed, first, period, float(value)) == 0
    return arr


def to_bf16(capi, arr):
    arr = np.ascontiguousarray(arr, np.float32)
    out = np.empty(arr.shape, np.uint16)
    assert capi.lib().tsm100_f32_to_bf16(arr.ctypes.data, out.ctypes.data, arr.size) == 0
    return out


def softmax_input(capi, rows, cols, seed=201):
    """3*N(0,1) with about 1 % of the positions set to +20 (the softmax configuration's law)."""
    x = gen_normal(capi, (rows, cols), seed, sigma=3.0)
    return plant_outliers(capi, x, seed + 1)


def f32_to_f16_bits(arr):
    return np.ascontiguousarray(arr, np.float32).astype(np.float16).view(np.uint16)


def dev_tensor(torch, arr):
    """Uploads a numpy array (uint16 arrays travel as int16) to cuda:0."""
    if arr.dtype == np.uint16:
        arr = arr.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(arr)).to("cuda:0")


def host_array(t, dtype=None):
    a = t.cpu().numpy()
    if dtype is not None:
        a = a.view(dtype)
    return a


def cur_stream(torch):
    return torch.cuda.current_stream().cuda_stream


def tol_16bit(ref_f32, significant_bits=8):
    """Element-wise absolute bound for a 16-bit result against the UNROUNDED f32 oracle:
    max(2e-2, half a unit in the last place of the storage type at |r| + 2^-9 * |r|).
    Rounding a correct f32 value to bf16 (8 significant bits) alone moves it by up to half an ulp,
    2^(floor(log2 |r|) - 8), which passes 2e-2 once |r| >= 8 (0.0156 on [4, 8), 0.031 on [8, 16));
    the 2^-9 * |r| term is one 16-bit rounding of an intermediate: the attention kernels hand the
    probabilities to the P V product in the storage type, and where one key dominates a row that
    rounding reaches the output undiminished (measured: 0.0045 at |r| = 4.1 with heads scaled by up to 4)."""
    ref = np.abs(np.asarray(ref_f32, np.float64))
    half_ulp = 2.0 ** (np.floor(np.log2(np.maximum(ref, 1e-30))) - significant_bits)
    return np.maximum(BF16_MAX_ABS, half_ulp + 2.0 ** -9 * ref)


def assert_16bit_close(oracle, got_f32, ref_f32, what="", report=False):
    """The 16-bit parity bar: relative Frobenius <= 1e-2 and, element-wise, |y - r| <= tol_16bit(r)
    against the unrounded f32 oracle.  Returns the metrics, with `over_2e-2` = how many elements
    differ by more than the flat 2e-2 (only ones with |r| >= 4 can, by rounding alone)."""
    m = oracle.compare(got_f32, ref_f32)
    assert m["rel_fro"] <= BF16_REL_FRO, (what, m)
    ref = np.asarray(ref_f32, np.float64)
    err = np.abs(np.asarray(got_f32, np.float64) - ref)
    tol = tol_16bit(ref)
    worst = float((err - tol).max())
    over = err > BF16_MAX_ABS
    m["over_2e-2"] = int(over.sum())
    m["over_2e-2_min_abs_ref"] = float(np.abs(ref[over]).min()) if over.any() else None
    if report:
        print(f"[parity] {what}: max_abs {m['max_abs']:.4g}, rel_fro {m['rel_fro']:.3g}, elements over 2e-2: "
              f"{m['over_2e-2']} of {err.size} (smallest |r| among them: {m['over_2e-2_min_abs_ref']})")
    assert worst <= 0, (what, m, worst)
    return m
