"""The CPU oracle against the committed float64 golden vectors, an independent
numpy statement, known answers and the edge cases of the domain."""
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle_np as onp

GOLD = Path(__file__).resolve().parent / "golden"


def test_softmax_matches_golden(oracle):
    g = np.load(GOLD / "softmax.npz")
    y = oracle.softmax_f32(g["x"])
    assert np.abs(y / g["y"] - 1).max() <= 2e-6  # f32 arithmetic against float64
    assert np.abs(oracle.softmax_f32(g["x"], f64_acc=True) / g["y"] - 1).max() <= 6.1e-8  # one f32 rounding


def test_gemm_matches_golden(oracle):
    g = np.load(GOLD / "gemm.npz")
    assert np.abs(oracle.gemm_f32(g["a"], g["b"]) - g["c"]).max() <= 2e-6
    assert np.abs(oracle.gemm_f32(g["a"], np.ascontiguousarray(g["b"].T), True) - g["c_t"]).max() <= 2e-6
    assert np.abs(oracle.gemm_f32(g["a"], g["b"], f64_acc=True) - g["c"]).max() <= 5e-7
    c32, c16 = oracle.gemm_bf16(g["a_bf16"], g["b_bf16"])
    assert np.abs(c32 - g["c_bf16"]).max() <= 2e-6
    assert np.array_equal(c16, onp.f32_to_bf16_bits(c32))


@pytest.mark.parametrize("key,heads,causal", [("o_gqa_causal", 4, True), ("o_gqa_full", 4, False),
                                              ("o_mha_full", 2, False), ("o_mha_causal", 2, True)])
def test_attention_matches_golden(oracle, key, heads, causal):
    g = np.load(GOLD / "attention.npz")
    q = np.ascontiguousarray(g["q"][:, :heads])
    o = oracle.attention_f32(q, g["k"], g["v"], causal)
    assert np.abs(o - g[key]).max() <= 2e-6


def test_attention_bf16_path_and_row_window(oracle):
    rng = np.random.default_rng(3)
    q, k, v = (oracle.f32_to_bf16(rng.standard_normal(s).astype(np.float32)) for s in ((1, 4, 40, 32), (1, 2, 40, 32), (1, 2, 40, 32)))
    o32, o16 = oracle.attention_bf16(q, k, v, True)
    ref = onp.attention(*(onp.bf16_bits_to_f32(t) for t in (q, k, v)), True)
    assert np.abs(o32 - ref).max() <= 2e-6
    assert np.array_equal(o16, onp.f32_to_bf16_bits(o32))
    w32, _ = oracle.attention_bf16(q, k, v, True, q_row0=17, q_rows=9)
    assert np.array_equal(w32, o32[:, :, 17:26])


def test_known_answers(oracle):
    # a constant row is uniform; one dominant entry takes all the mass
    y = oracle.softmax_f32(np.full((2, 7), 3.25, np.float32))
    assert np.allclose(y, 1.0 / 7.0, rtol=0, atol=1e-8)
    x = np.zeros((1, 5), np.float32)
    x[0, 2] = 200.0
    assert np.array_equal(oracle.softmax_f32(x), np.array([[0, 0, 1, 0, 0]], np.float32))
    # identity and zero contraction
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    assert np.array_equal(oracle.gemm_f32(a, np.eye(4, dtype=np.float32)), a)
    assert np.array_equal(oracle.gemm_f32(np.zeros((3, 0), np.float32), np.zeros((0, 2), np.float32)), np.zeros((3, 2), np.float32))
    # causal attention: the first query row sees only the first key, so it returns V[0]
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((1, 1, 6, 8)).astype(np.float32) for _ in range(3))
    o = oracle.attention_f32(q, k, v, True)
    assert np.array_equal(o[0, 0, 0], v[0, 0, 0])
    # identical keys: attention is the mean of V
    k[:] = k[0, 0, 0]
    o = oracle.attention_f32(q, k, v, False)
    assert np.abs(o[0, 0] - v[0, 0].mean(axis=0)).max() <= 1e-6


def test_bf16_rounding_is_nearest_even(oracle):
    vals = np.array([1.0, 1.00390625, 1.005859375, 1.01171875, -2.5, 3.0e38, 1e-40, 0.0], np.float32)
    # 1.00390625 = 1 + 2^-8 is a tie -> rounds to even (1.0); 1.01171875 = 1 + 3*2^-8 is a tie -> 1.015625
    got = oracle.bf16_to_f32(oracle.f32_to_bf16(vals))
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == 1.0078125 and got[3] == 1.015625 and got[4] == -2.5
    assert np.array_equal(oracle.f32_to_bf16(vals), onp.f32_to_bf16_bits(vals))
    rng = np.random.default_rng(5)
    r = rng.standard_normal(10000).astype(np.float32) * 100
    assert np.array_equal(oracle.f32_to_bf16(r), onp.f32_to_bf16_bits(r))
    assert np.array_equal(oracle.bf16_to_f32(oracle.f32_to_bf16(r)), onp.bf16_bits_to_f32(onp.f32_to_bf16_bits(r)))


def test_softmax_outliers_and_random_against_numpy(oracle, pkg):
    import util
    x = util.softmax_input(pkg.capi, 40, 1000)
    y = oracle.softmax_f32(x)
    ref = onp.softmax(x)
    assert np.abs(y / ref - 1).max() <= 1e-5
    # about 1 % of the positions are +20 and they carry nearly all the mass
    hot = x == 20.0
    assert 0.005 < hot.mean() < 0.02
    assert (y * hot).sum(axis=1).min() > 0.9
    xb = util.to_bf16(pkg.capi, x)
    y32, y16 = oracle.softmax_bf16(xb)
    assert np.abs(y32 - onp.softmax(onp.bf16_bits_to_f32(xb))).max() <= 1e-6
    assert np.array_equal(y16, onp.f32_to_bf16_bits(y32))


def test_compare_metrics(oracle):
    r = np.array([1.0, -2.0, 4.0, 0.0], np.float32)
    y = np.array([1.5, -2.0, 4.0, 0.0], np.float32)
    m = oracle.compare(y, r, floor_r=0.5)
    assert m["max_abs"] == 0.5 and m["max_ref"] == 4.0 and m["rel_max"] == 0.125
    assert abs(m["rel_fro"] - 0.5 / np.sqrt(21.0)) < 1e-12 and m["max_elem_rel"] == 0.5


def test_row_operators_match_golden(oracle):
    g = np.load(GOLD / "rowops.npz")
    x, eps = g["x"], float(g["eps"])
    assert np.abs(oracle.rms_norm_f32(x, eps) / g["rms"] - 1).max() <= 2e-6
    assert np.abs(oracle.rms_norm_f32(x, eps, f64_acc=True) / g["rms"] - 1).max() <= 6.1e-8
    assert np.abs(oracle.reduce_f32(x, "sum") - g["row_sum"]).max() <= 2e-4   # 96 terms of size ~3 in f32
    assert np.abs(oracle.reduce_f32(x, "sum", f64_acc=True) - g["row_sum"]).max() <= 2e-6
    assert np.array_equal(oracle.reduce_f32(x, "max"), g["row_max"].astype(np.float32))
    def rel(a, ref):  # error relative to the largest magnitude (values reach ~15 and ~40 here)
        return np.abs(a - ref).max() / np.abs(ref).max()
    assert rel(oracle.silu_mul_f32(g["gate"], None), g["silu"]) <= 2e-7       # f32 exp and divide against float64
    assert rel(oracle.silu_mul_f32(g["gate"], g["up"]), g["silu_mul"]) <= 2e-7
    assert rel(oracle.silu_mul_f32(g["gate"], g["up"], f64_acc=True), g["silu_mul"]) <= 6.1e-8  # one f32 rounding


def test_row_operators_known_answers_and_bf16(oracle):
    # a row of equal magnitudes normalises to +-1 (eps = 0); scaling the input leaves rms_norm unchanged
    x = np.array([[2.0, -2.0, 2.0, -2.0], [0.5, 0.5, 0.5, 0.5]], np.float32)
    assert np.array_equal(oracle.rms_norm_f32(x, 0.0), np.sign(x))
    rng = np.random.default_rng(11)
    r = rng.standard_normal((5, 64)).astype(np.float32)
    assert np.abs(oracle.rms_norm_f32(r, 0.0) - oracle.rms_norm_f32(4.0 * r, 0.0)).max() <= 1e-6
    # an all-zero row: rsqrt(eps) * 0 = 0
    assert np.array_equal(oracle.rms_norm_f32(np.zeros((1, 8), np.float32), 1e-6), np.zeros((1, 8), np.float32))
    # empty rows: the fill values of the reductions
    e = np.zeros((3, 0), np.float32)
    assert np.array_equal(oracle.reduce_f32(e, "sum"), np.zeros(3, np.float32))
    assert np.all(np.isneginf(oracle.reduce_f32(e, "max")))
    # silu: 0 -> 0, large positive -> x, large negative -> -0
    s = oracle.silu_mul_f32(np.array([0.0, 50.0, -200.0], np.float32), None)
    assert s[0] == 0.0 and s[1] == 50.0 and s[2] == 0.0
    # bf16 I/O: widen, f32 math, one RNE rounding
    xb = oracle.f32_to_bf16(r)
    y32, y16 = oracle.rms_norm_bf16(xb, 1e-5)
    assert np.abs(y32 - onp.rms_norm(onp.bf16_bits_to_f32(xb), 1e-5)).max() <= 2e-6
    assert np.array_equal(y16, onp.f32_to_bf16_bits(y32))
    gb, ub = oracle.f32_to_bf16(3 * r), oracle.f32_to_bf16(r[::-1].copy())
    s32, s16 = oracle.silu_mul_bf16(gb, ub)
    assert np.abs(s32 - onp.silu_mul(onp.bf16_bits_to_f32(gb), onp.bf16_bits_to_f32(ub))).max() <= 2e-6
    assert np.array_equal(s16, onp.f32_to_bf16_bits(s32))


def test_attention_decode_matches_golden_and_known_answers(oracle):
    g = np.load(GOLD / "attention_decode.npz")
    n = int(g["seq_len"])
    assert np.abs(oracle.attention_decode_f32(g["q"], g["k_cache"], g["v_cache"], n) - g["o"]).max() <= 2e-6
    assert np.abs(oracle.attention_decode_f32(g["q"], g["k_cache"], g["v_cache"], n, f64_acc=True) - g["o"]).max() <= 3e-7
    # the unfilled part of the cache is never read
    k2, v2 = g["k_cache"].copy(), g["v_cache"].copy()
    k2[:, :, n:], v2[:, :, n:] = np.nan, np.nan
    assert np.array_equal(oracle.attention_decode_f32(g["q"], k2, v2, n), oracle.attention_decode_f32(g["q"], g["k_cache"], g["v_cache"], n))
    # one filled position returns its V row; identical keys average V; decode equals the last row of causal attention
    assert np.array_equal(oracle.attention_decode_f32(g["q"], g["k_cache"], g["v_cache"], 1)[:, :2], g["v_cache"][:, :, 0][:, [0, 0]])
    rng = np.random.default_rng(4)
    q, k, v = (rng.standard_normal(s).astype(np.float32) for s in ((1, 3, 12, 8), (1, 3, 12, 8), (1, 3, 12, 8)))
    full = oracle.attention_f32(q, k, v, True)
    dec = oracle.attention_decode_f32(np.ascontiguousarray(q[:, :, -1]), k, v, 12)
    assert np.abs(dec - full[:, :, -1]).max() <= 1e-6
    qb, kb, vb = (oracle.f32_to_bf16(t) for t in (np.ascontiguousarray(q[:, :, -1]), k, v))
    o32, o16 = oracle.attention_decode_bf16(qb, kb, vb, 12)
    assert np.abs(o32 - onp.attention_decode(*(onp.bf16_bits_to_f32(t) for t in (qb, kb, vb)), 12)).max() <= 2e-6
    assert np.array_equal(o16, onp.f32_to_bf16_bits(o32))


def test_rope_and_kv_cache_update(oracle):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 6, 3, 32)).astype(np.float32)
    ref = onp.rope(x, 11, 10000.0)
    assert np.abs(oracle.rope_f32(x, 11, 10000.0) - ref).max() <= 5e-6   # f32 pow / cos / sin at angles up to 16
    assert np.abs(oracle.rope_f32(x, 11, 10000.0, f64_acc=True) - ref).max() <= 3e-7
    # position 0 is the identity; a rotation keeps the norm of every pair
    assert np.array_equal(oracle.rope_f32(x[:, :1], 0, 10000.0), x[:, :1])
    y = oracle.rope_f32(x, 100, 500000.0)
    assert np.abs((y[..., 0::2] ** 2 + y[..., 1::2] ** 2) - (x[..., 0::2] ** 2 + x[..., 1::2] ** 2)).max() <= 1e-5
    # decode form = prefill form of one token at that position
    assert np.array_equal(oracle.rope_f32(x, 11, 10000.0)[:, 4:5], oracle.rope_f32(x[:, 4:5], 15, 10000.0))
    src = rng.standard_normal((2, 3, 4, 8)).astype(np.float32)
    cache = rng.standard_normal((2, 4, 10, 8)).astype(np.float32)
    out = oracle.kv_cache_update(src, cache, 5)
    assert np.array_equal(out[:, :, 5:8], src.transpose(0, 2, 1, 3))
    assert np.array_equal(out[:, :, :5], cache[:, :, :5]) and np.array_equal(out[:, :, 8:], cache[:, :, 8:])
    s16 = oracle.f32_to_bf16(src)
    assert np.array_equal(oracle.kv_cache_update(s16, np.zeros((2, 4, 10, 8), np.uint16), 0)[:, :, :3], s16.transpose(0, 2, 1, 3))


def test_attention_prefill_oracle(oracle):
    rng = np.random.default_rng(9)
    s, hq, hkv, d, start, max_seq = 7, 4, 2, 16, 5, 16
    q = rng.standard_normal((s, hq, d)).astype(np.float32)
    k, v = (rng.standard_normal((hkv, max_seq, d)).astype(np.float32) for _ in range(2))
    o = oracle.attention_prefill_f32(q, k, v, start)
    # token i of the prefill is a decode step against the first start + i + 1 positions
    for i in range(s):
        dec = oracle.attention_decode_f32(q[None, i], k[None], v[None], start + i + 1)
        assert np.abs(o[i] - dec[0]).max() <= 1e-6
    assert np.abs(oracle.attention_prefill_f32(q, k, v, start, f64_acc=True) - o).max() <= 2e-6
    # start_pos 0 with the cache equal to K / V is plain causal attention in the other layout
    full = oracle.attention_f32(np.ascontiguousarray(q.transpose(1, 0, 2))[None], k[None, :, :s], v[None, :, :s], True)
    assert np.abs(oracle.attention_prefill_f32(q, k, v, 0) - full[0].transpose(1, 0, 2)).max() <= 1e-6
