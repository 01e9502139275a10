"""Single-token attention against a KV cache on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def run_decode(dev, capi, q, k, v, seq_len, dtype):
    b, hq, d = q.shape
    _, hkv, max_seq, _ = k.shape
    qd, kd, vd = (util.dev_tensor(torch, t) for t in (q, k, v))
    od = torch.full_like(qd, 12345 if qd.dtype == torch.int16 else float("nan"))
    dev.attention_decode(dtype, b, hq, hkv, seq_len, max_seq, d, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), od.data_ptr(),
                         stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    return od.cpu().numpy()


# (batch, heads_q, heads_kv, seq_len, max_seq, head_dim): group sizes 1, 2, 3 (padded to 4), 8 and 12 (two passes);
# ranges that end inside a warp's slots; one position; long caches that are split over a cluster
CASES = [(1, 1, 1, 1, 8, 64), (2, 4, 4, 33, 40, 128), (1, 8, 4, 100, 128, 64), (2, 6, 2, 257, 300, 128), (1, 16, 2, 1000, 1024, 128),
         (1, 24, 2, 515, 600, 64), (3, 8, 1, 4096, 4096, 128), (1, 2, 2, 20000, 20480, 128), (1, 8, 1, 16384, 16384, 64),
         (2, 10, 2, 77, 80, 128), (1, 40, 2, 1029, 1100, 64)]  # f32 groups of 5 and 20 (two passes): tensor cores, three TF32 products


@pytest.mark.parametrize("b,hq,hkv,n,max_seq,d", CASES)
def test_decode_f32_matches_oracle(dev, pkg, oracle, b, hq, hkv, n, max_seq, d):
    capi = pkg.capi
    q = util.gen_normal(capi, (b, hq, d), 801)
    k = util.gen_normal(capi, (b, hkv, max_seq, d), 802)
    v = util.gen_normal(capi, (b, hkv, max_seq, d), 803)
    k[:, :, n:], v[:, :, n:] = np.nan, np.nan  # positions beyond seq_len must not be read
    o = run_decode(dev, capi, q, k, v, n, capi.F32)
    kz, vz = np.nan_to_num(k), np.nan_to_num(v)
    for ref in (oracle.attention_decode_f32(q, kz, vz, n), oracle.attention_decode_f32(q, kz, vz, n, f64_acc=True)):
        m = oracle.compare(o, ref)
        assert m["rel_max"] <= util.F32_REL and m["rel_fro"] <= util.F32_REL, m


@pytest.mark.parametrize("b,hq,hkv,n,max_seq,d", [(1, 1, 1, 5, 8, 64), (2, 8, 2, 300, 320, 128), (1, 32, 4, 2048, 2048, 128),
                                                     (2, 5, 1, 777, 800, 64), (1, 8, 8, 9000, 9000, 128),
                                                     # few caches, long: eight-warp CTAs in clusters of 16 (ragged last range)
                                                     (1, 16, 2, 8207, 8208, 128), (1, 4, 4, 8192, 8192, 64)])
def test_decode_bf16_matches_oracle(dev, pkg, oracle, b, hq, hkv, n, max_seq, d):
    capi = pkg.capi
    q = util.to_bf16(capi, util.gen_normal(capi, (b, hq, d), 801))
    k = util.to_bf16(capi, util.gen_normal(capi, (b, hkv, max_seq, d), 802))
    v = util.to_bf16(capi, util.gen_normal(capi, (b, hkv, max_seq, d), 803))
    o = run_decode(dev, capi, q, k, v, n, capi.BF16).view(np.uint16)
    ref32, _ = oracle.attention_decode_bf16(q, k, v, n)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)


def test_decode_f16_and_large_scores(dev, pkg, oracle):
    capi = pkg.capi
    q = util.f32_to_f16_bits(8.0 * util.gen_normal(capi, (1, 4, 128), 811))   # scores of a few hundred: max subtraction matters
    k = util.f32_to_f16_bits(util.gen_normal(capi, (1, 2, 600, 128), 812))
    v = util.f32_to_f16_bits(util.gen_normal(capi, (1, 2, 600, 128), 813))
    o = run_decode(dev, capi, q, k, v, 600, capi.F16).view(np.float16).astype(np.float32)
    f = lambda t: t.view(np.float16).astype(np.float32)
    ref = oracle.attention_decode_f32(f(q), f(k), f(v), 600, f64_acc=True)
    assert np.abs(o - ref).max() <= 2.0 ** -10 * max(1.0, float(np.abs(ref).max())) + 1e-3


def test_decode_equals_last_row_of_causal_attention(dev, pkg, oracle):
    """Size-independent property at a full-size cache: decoding the last token of a sequence reproduces the
    last row of the fused causal attention over the same keys and values."""
    capi = pkg.capi
    b, hq, hkv, s, d = 1, 8, 2, 4096, 128
    q = util.to_bf16(capi, util.gen_normal(capi, (b, hq, s, d), 821))
    k = util.to_bf16(capi, util.gen_normal(capi, (b, hkv, s, d), 822))
    v = util.to_bf16(capi, util.gen_normal(capi, (b, hkv, s, d), 823))
    qd, kd, vd = (util.dev_tensor(torch, t) for t in (q, k, v))
    full = torch.empty_like(qd)
    dev.attention(capi.BF16, b, hq, hkv, s, d, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), full.data_ptr(), causal=True,
                  stream=util.cur_stream(torch))
    last_q = qd[:, :, -1].contiguous()
    dec = torch.empty_like(last_q)
    dev.attention_decode(capi.BF16, b, hq, hkv, s, s, d, last_q.data_ptr(), kd.data_ptr(), vd.data_ptr(), dec.data_ptr(),
                         stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    a = oracle.bf16_to_f32(full[:, :, -1].contiguous().cpu().numpy().view(np.uint16))
    c = oracle.bf16_to_f32(dec.cpu().numpy().view(np.uint16))
    assert np.abs(a - c).max() <= 2.0 ** -7  # two independently rounded bf16 results of values below one


def test_decode_rejects_bad_arguments(dev, pkg):
    capi = pkg.capi
    with pytest.raises(pkg.hal.HalError):
        dev.attention_decode(capi.F32, 1, 4, 3, 8, 8, 64, 16, 16, 16, 16)      # heads_q not a multiple of heads_kv
    with pytest.raises(pkg.hal.HalError):
        dev.attention_decode(capi.F32, 1, 4, 4, 9, 8, 64, 16, 16, 16, 16)      # seq_len beyond the cache
    with pytest.raises(pkg.hal.HalError):
        dev.attention_decode(capi.F32, 1, 4, 4, 8, 8, 80, 16, 16, 16, 16)      # head_dim
    with pytest.raises(pkg.hal.HalError):
        dev.attention_decode(capi.F32, 1, 4, 4, 8, 8, 64, 0, 16, 16, 16)       # null q


def rope_tol(x, last_pos):
    """f32 pow / sin / cos differ between libraries by a few ulp; an ulp of the angle is worth |angle| * 6e-8 of
    the rotated values, so the bound grows with the position."""
    return (1e-6 + 4e-7 * last_pos) * float(np.abs(x).max())


@pytest.mark.parametrize("b,s,h,d,start,theta", [(1, 1, 1, 2, 0, 10000.0), (2, 1, 8, 128, 777, 10000.0), (1, 37, 5, 64, 3, 10000.0),
                                                   (2, 300, 4, 128, 1000, 500000.0), (1, 4, 3, 6, 0, 100.0)])
def test_rope_f32_matches_oracle(dev, pkg, oracle, b, s, h, d, start, theta):
    capi = pkg.capi
    x = util.gen_normal(capi, (b, s, h, d), 901)
    xd = util.dev_tensor(torch, x)
    dev.rope(capi.F32, b, s, h, d, start, theta, xd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    got = xd.cpu().numpy()
    tol = rope_tol(x, start + s)
    assert np.abs(got - oracle.rope_f32(x, start, theta)).max() <= tol
    assert np.abs(got - oracle.rope_f32(x, start, theta, f64_acc=True)).max() <= tol
    # rotations keep the norm of every pair whatever the angle
    assert np.abs((got[..., 0::2] ** 2 + got[..., 1::2] ** 2) - (x[..., 0::2] ** 2 + x[..., 1::2] ** 2)).max() <= 1e-5 * float((x ** 2).max() * 2)


def test_rope_bf16(dev, pkg, oracle):
    capi = pkg.capi
    xb = util.to_bf16(capi, util.gen_normal(capi, (2, 9, 4, 128), 902))
    xd = util.dev_tensor(torch, xb)
    dev.rope(capi.BF16, 2, 9, 4, 128, 50, 10000.0, xd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    got = oracle.bf16_to_f32(xd.cpu().numpy().view(np.uint16))
    ref = oracle.rope_f32(oracle.bf16_to_f32(xb), 50, 10000.0, f64_acc=True)
    util.assert_16bit_close(oracle, got, ref)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("b,s,h,d,start,max_seq", [(1, 1, 1, 8, 0, 1), (2, 1, 8, 128, 41, 64), (2, 33, 4, 64, 7, 40), (1, 5, 3, 6, 2, 9)])
def test_kv_cache_update_is_exact(dev, pkg, oracle, dt, b, s, h, d, start, max_seq):
    capi = pkg.capi
    src = util.gen_normal(capi, (b, s, h, d), 903)
    cache = util.gen_normal(capi, (b, h, max_seq, d), 904)
    code = capi.F32
    if dt == "bf16":
        src, cache, code = util.to_bf16(capi, src), util.to_bf16(capi, cache), capi.BF16
    sd, cd = util.dev_tensor(torch, src), util.dev_tensor(torch, cache)
    dev.kv_cache_update(code, b, s, h, d, start, max_seq, sd.data_ptr(), cd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    got = cd.cpu().numpy().view(src.dtype)
    assert np.array_equal(got, oracle.kv_cache_update(src, cache, start))
    with pytest.raises(pkg.hal.HalError):
        dev.kv_cache_update(code, b, s, h, d, max_seq, max_seq, sd.data_ptr(), cd.data_ptr())  # would write past the cache


def test_decode_step_chain(dev, pkg, oracle):
    """rope(q), rope(k), append k and v to the caches, attend: one decode step through the C ABI against the same
    chain in the oracle."""
    capi = pkg.capi
    b, hq, hkv, d, pos, max_seq, theta = 2, 8, 2, 128, 300, 512, 10000.0
    q = util.gen_normal(capi, (b, 1, hq, d), 911)
    k_new, v_new = util.gen_normal(capi, (b, 1, hkv, d), 912), util.gen_normal(capi, (b, 1, hkv, d), 913)
    kc, vc = util.gen_normal(capi, (b, hkv, max_seq, d), 914), util.gen_normal(capi, (b, hkv, max_seq, d), 915)
    qd, knd, vnd, kcd, vcd = (util.dev_tensor(torch, t) for t in (q, k_new, v_new, kc, vc))
    od = torch.empty(b, hq, d, device="cuda:0")
    s = util.cur_stream(torch)
    dev.rope(capi.F32, b, 1, hq, d, pos, theta, qd.data_ptr(), stream=s)
    dev.rope(capi.F32, b, 1, hkv, d, pos, theta, knd.data_ptr(), stream=s)
    dev.kv_cache_update(capi.F32, b, 1, hkv, d, pos, max_seq, knd.data_ptr(), kcd.data_ptr(), stream=s)
    dev.kv_cache_update(capi.F32, b, 1, hkv, d, pos, max_seq, vnd.data_ptr(), vcd.data_ptr(), stream=s)
    dev.attention_decode(capi.F32, b, hq, hkv, pos + 1, max_seq, d, qd.data_ptr(), kcd.data_ptr(), vcd.data_ptr(), od.data_ptr(), stream=s)
    torch.cuda.synchronize()
    qr, kr = oracle.rope_f32(q, pos, theta, f64_acc=True), oracle.rope_f32(k_new, pos, theta, f64_acc=True)
    ref = oracle.attention_decode_f32(qr[:, 0], oracle.kv_cache_update(kr, kc, pos), oracle.kv_cache_update(v_new, vc, pos), pos + 1,
                                      f64_acc=True)
    assert np.abs(od.cpu().numpy() - ref).max() <= 2e-4 * float(np.abs(ref).max())  # rope at position 300 in f32 dominates
    assert dev.status() == 0


def run_prefill(dev, capi, q, k, v, start, dtype):
    s, hq, d = q.shape
    hkv, max_seq, _ = k.shape
    qd, kd, vd = (util.dev_tensor(torch, t) for t in (q, k, v))
    od = torch.full_like(qd, 12345 if qd.dtype == torch.int16 else float("nan"))
    dev.attention_prefill(dtype, hq, hkv, s, start, max_seq, d, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), od.data_ptr(),
                          stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    return od.cpu().numpy()


@pytest.mark.parametrize("s,hq,hkv,d,start,max_seq", [(1, 1, 1, 64, 0, 4), (7, 4, 2, 64, 5, 16), (130, 6, 3, 128, 0, 130),
                                                        (33, 8, 2, 96, 100, 200), (256, 2, 2, 128, 300, 600)])
def test_prefill_f32_matches_oracle(dev, pkg, oracle, s, hq, hkv, d, start, max_seq):
    capi = pkg.capi
    q = util.gen_normal(capi, (s, hq, d), 921)
    k, v = util.gen_normal(capi, (hkv, max_seq, d), 922), util.gen_normal(capi, (hkv, max_seq, d), 923)
    k[:, start + s:], v[:, start + s:] = np.nan, np.nan  # beyond the filled part: must not be read
    o = run_prefill(dev, capi, q, k, v, start, capi.F32)
    kz, vz = np.nan_to_num(k), np.nan_to_num(v)
    for ref in (oracle.attention_prefill_f32(q, kz, vz, start), oracle.attention_prefill_f32(q, kz, vz, start, f64_acc=True)):
        m = oracle.compare(o, ref)
        assert m["rel_max"] <= util.F32_REL and m["rel_fro"] <= util.F32_REL, m


# tensor-core path: offsets that are and are not multiples of the 128-key step, ragged lengths, grouped heads
@pytest.mark.parametrize("s,hq,hkv,start,max_seq", [(1, 2, 2, 0, 8), (256, 4, 2, 0, 256), (200, 8, 2, 100, 512), (384, 2, 1, 128, 600),
                                                      (130, 4, 4, 1000, 1200), (1024, 4, 1, 77, 2048)])
def test_prefill_bf16_tensor_core(dev, pkg, oracle, s, hq, hkv, start, max_seq):
    capi = pkg.capi
    d = 128
    q = util.to_bf16(capi, util.gen_normal(capi, (s, hq, d), 921))
    k = util.to_bf16(capi, util.gen_normal(capi, (hkv, max_seq, d), 922))
    v = util.to_bf16(capi, util.gen_normal(capi, (hkv, max_seq, d), 923))
    o = run_prefill(dev, capi, q, k, v, start, capi.BF16).view(np.uint16)
    f = oracle.bf16_to_f32
    ref = oracle.attention_prefill_f32(f(q), f(k), f(v), start)
    util.assert_16bit_close(oracle, f(o), ref)


def test_prefill_in_chunks_equals_one_shot_and_plain_causal(dev, pkg, oracle):
    """Size-independent properties at seq 2048: prefill from position 0 reproduces plain causal attention over the
    same K / V, and prefilling the second half on top of the first gives the same rows."""
    capi = pkg.capi
    s, hq, hkv, d = 2048, 4, 2, 128
    q = util.to_bf16(capi, util.gen_normal(capi, (s, hq, d), 931))
    k = util.to_bf16(capi, util.gen_normal(capi, (hkv, s, d), 932))
    v = util.to_bf16(capi, util.gen_normal(capi, (hkv, s, d), 933))
    one = run_prefill(dev, capi, q, k, v, 0, capi.BF16)
    second = run_prefill(dev, capi, np.ascontiguousarray(q[s // 2:]), k, v, s // 2, capi.BF16)
    assert np.array_equal(second, one[s // 2:])  # same tiles, same arithmetic
    qh = util.dev_tensor(torch, np.ascontiguousarray(q.transpose(1, 0, 2))[None])
    kd, vd = util.dev_tensor(torch, k[None]), util.dev_tensor(torch, v[None])
    full = torch.empty_like(qh)
    dev.attention(capi.BF16, 1, hq, hkv, s, d, qh.data_ptr(), kd.data_ptr(), vd.data_ptr(), full.data_ptr(), causal=True,
                  stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert np.array_equal(full.cpu().numpy()[0].transpose(1, 0, 2), one)
