"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the
header declares, fails loudly instead of falling back, and its host-only parts
(sharding, input generator) are correct."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import util

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "tile_sm100.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tsm100_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.capi.lib()
    names = declared_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in tile_sm100.h but not exported"
    # and the Python binding declares a prototype for each of them
    assert sorted(pkg.capi.PROTOTYPES) == names
    assert lib.tsm100_version() == 100
    assert lib.tsm100_target_name() == b"cuda_sm100" and lib.tsm100_target_ext() == b"cu"


def test_no_device_is_an_error_not_a_fallback(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib, capi = pkg.capi.lib(), pkg.capi
    n = C.c_int32(-1)
    assert lib.tsm100_device_count(C.byref(n)) == capi.ERR_NO_DEVICE
    h = C.c_void_p()
    assert lib.tsm100_device_open(0, C.byref(h)) == capi.ERR_NO_DEVICE and not h.value
    assert "failed" in capi.last_error()
    with pytest.raises(pkg.hal.BackendNotAvailable):
        pkg.hal.CudaSm100Device(0)
    # compute entry points reject a null device handle instead of computing on the host
    d = capi.SoftmaxDesc(capi.F32, 1, 4)
    x = np.zeros(4, np.float32)
    assert lib.tsm100_softmax(None, C.byref(d), x.ctypes.data, x.ctypes.data, None) == capi.ERR_INVALID
    assert lib.tsm100_softmax_host(None, C.byref(d), x.ctypes.data, x.ctypes.data) == capi.ERR_INVALID
    assert np.array_equal(x, np.zeros(4, np.float32))


def test_shard_range(pkg):
    sh = pkg.launcher
    for units in (0, 1, 7, 16, 64, 65536, 100003):
        for world in (1, 2, 3, 4, 8):
            parts = [sh.shard_range(units, world, r) for r in range(world)]
            assert parts[0].first == 0 and parts[-1].stop == units
            assert all(parts[i].stop == parts[i + 1].first for i in range(world - 1))
            counts = [p.count for p in parts]
            assert max(counts) - min(counts) <= 1 and counts == sorted(counts, reverse=True)
    with pytest.raises(ValueError):
        sh.shard_range(8, 0, 0)
    with pytest.raises(ValueError):
        sh.shard_range(8, 4, 4)
    # the configurations' partitions on an 8-GPU box
    assert [sh.shard_range(65536, 8, r).count for r in range(8)] == [8192] * 8     # softmax rows
    assert [sh.shard_range(64, 8, r).count for r in range(8)] == [8] * 8           # GEMM problems of the batch
    assert [sh.shard_range(8 * 32, 8, r).count for r in range(8)] == [32] * 8      # (batch, head) groups
    assert [(s.first, s.count) for s in (sh.shard_range(2 * 8, 8, r) for r in range(8))] == [(2 * r, 2) for r in range(8)]
    # (the N-column split of one large GEMM is a launcher plan: tests/test_launcher.py)


def _splitmix(z):
    m = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def _draw(seed, i):
    return _splitmix(seed ^ ((i * 0x9E3779B97F4A7C15) & ((1 << 64) - 1)))


def test_generator_matches_its_definition_and_golden(pkg):
    capi = pkg.capi
    u = util.gen_uniform(capi, (50,), 101)
    want = np.array([(_draw(101, i) >> 40) * (2.0 / 16777216.0) - 1.0 for i in range(50)], np.float32)
    assert np.array_equal(u, want)
    z = util.gen_normal(capi, (50,), 201, 3.0)
    ref = []
    for i in range(50):
        p = i >> 1
        u1 = ((_draw(201, 2 * p) >> 40) + 1.0) / 16777216.0
        u2 = (_draw(201, 2 * p + 1) >> 40) / 16777216.0
        r = np.sqrt(-2.0 * np.log(u1))
        ref.append(3.0 * r * (np.sin(2 * np.pi * u2) if i & 1 else np.cos(2 * np.pi * u2)))
    assert np.abs(z - np.array(ref, np.float32)).max() <= 1e-6
    # sub-ranges reproduce the same stream (each rank generates only its shard)
    assert np.array_equal(util.gen_normal(capi, (20,), 201, 3.0, first=30), z[30:50])
    assert np.array_equal(util.gen_uniform(capi, (10,), 101, first=40), u[40:50])
    g = np.load(Path(__file__).resolve().parent / "golden" / "generator.npz")
    assert np.array_equal(util.gen_uniform(capi, (64,), 101), g["uniform_101"])
    assert np.abs(util.gen_normal(capi, (64,), 201, 3.0) - g["normal_201"]).max() <= 1e-6
    assert np.abs(util.gen_normal(capi, (16,), 201, 3.0, first=1000) - g["normal_201_from_1000"]).max() <= 1e-6
    hot = util.plant_outliers(capi, np.zeros(2000, np.float32), 202).nonzero()[0]
    assert np.array_equal(hot, g["outliers_202"])
    assert np.array_equal(hot, np.array([i for i in range(2000) if _draw(202, i) % 100 == 0]))
    # the bf16 form is the same stream, scaled and rounded once
    direct = np.empty(33, np.uint16)
    assert capi.lib().tsm100_fill_normal_bf16(direct.ctypes.data, direct.size, 201, 17, 3.0, 0.5) == 0
    assert np.array_equal(direct, util.to_bf16(capi, util.gen_normal(capi, (33,), 201, 3.0, first=17) * np.float32(0.5)))
    big = util.gen_normal(capi, (200000,), 7)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1.0) < 0.01


def test_bf16_conversion_matches_oracle(pkg, oracle):
    x = util.gen_normal(pkg.capi, (4096,), 9, 50.0)
    b = util.to_bf16(pkg.capi, x)
    assert np.array_equal(b, oracle.f32_to_bf16(x))
    back = np.empty(x.shape, np.float32)
    assert pkg.capi.lib().tsm100_bf16_to_f32(b.ctypes.data, back.ctypes.data, b.size) == 0
    assert np.array_equal(back, oracle.bf16_to_f32(b))
