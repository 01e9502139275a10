"""Fused attention forward on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def run_attention(dev, capi, q, k, v, dtype, causal):
    b, hq, s, d = q.shape
    qd, kd, vd = (util.dev_tensor(torch, t) for t in (q, k, v))
    od = torch.full_like(qd, 12345 if qd.dtype == torch.int16 else float("nan"))
    dev.attention(dtype, b, hq, k.shape[1], s, d, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), od.data_ptr(),
                  causal=causal, stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    return od.cpu().numpy()


def bf16_qkv(capi, b, hq, hkv, s, d, seed=401):
    q = util.to_bf16(capi, util.gen_normal(capi, (b, hq, s, d), seed))
    k = util.to_bf16(capi, util.gen_normal(capi, (b, hkv, s, d), seed + 1))
    v = util.to_bf16(capi, util.gen_normal(capi, (b, hkv, s, d), seed + 2))
    return q, k, v


TC_CASES = [
    (1, 1, 1, 128), (1, 1, 1, 256), (1, 2, 2, 512), (2, 2, 2, 384),   # 384: second query tile half empty
    (1, 2, 2, 200), (1, 1, 1, 1000),                                    # ragged tails
    (1, 8, 2, 512), (2, 4, 1, 768),                                     # grouped KV heads
    (1, 2, 2, 2048),
]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,hq,hkv,s", TC_CASES)
def test_attention_bf16_tensor_core(dev, pkg, oracle, b, hq, hkv, s, causal):
    capi = pkg.capi
    q, k, v = bf16_qkv(capi, b, hq, hkv, s, 128)
    o = run_attention(dev, capi, q, k, v, capi.BF16, causal).view(np.uint16)
    ref32, _ = oracle.attention_bf16(q, k, v, causal)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)


def test_attention_gqa_scaled_heads(dev, pkg, oracle):
    """Per-head scales in [0.5, 2] on Q and K/V (the grouped-query configuration's law), causal."""
    capi = pkg.capi
    b, hq, hkv, s, d = 1, 8, 2, 1024, 128
    qf = util.gen_normal(capi, (b, hq, s, d), 501)
    kf = util.gen_normal(capi, (b, hkv, s, d), 502)
    vf = util.gen_normal(capi, (b, hkv, s, d), 503)
    uq = 0.5 + 0.75 * (util.gen_uniform(capi, (hq,), 504) + 1.0)
    ukv = 0.5 + 0.75 * (util.gen_uniform(capi, (hkv,), 504, first=hq) + 1.0)
    qf *= uq[None, :, None, None]
    kf *= ukv[None, :, None, None]
    vf *= ukv[None, :, None, None]
    q, k, v = (util.to_bf16(capi, t) for t in (qf, kf, vf))
    o = run_attention(dev, capi, q, k, v, capi.BF16, True).view(np.uint16)
    ref32, _ = oracle.attention_bf16(q, k, v, True)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_f32_fp32_pipe(dev, pkg, oracle, causal):
    capi = pkg.capi
    b, hq, hkv, s, d = 2, 4, 2, 100, 64
    q = util.gen_normal(capi, (b, hq, s, d), 411)
    k = util.gen_normal(capi, (b, hkv, s, d), 412)
    v = util.gen_normal(capi, (b, hkv, s, d), 413)
    o = run_attention(dev, capi, q, k, v, capi.F32, causal)
    m = oracle.compare(o, oracle.attention_f32(q, k, v, causal))
    assert m["rel_max"] <= 1e-5 and m["rel_fro"] <= 1e-5, m


@pytest.mark.parametrize("b,hq,hkv,s,d,causal", [(1, 2, 2, 333, 128, False), (1, 4, 2, 333, 128, True), (2, 2, 1, 64, 64, True),
                                                    (1, 1, 1, 1, 128, True), (1, 2, 2, 700, 64, False), (1, 3, 3, 129, 128, True),
                                                    (1, 2, 1, 200, 96, True), (2, 2, 2, 150, 32, False)])
def test_attention_f32_tensor_core_three_tf32(dev, pkg, oracle, b, hq, hkv, s, d, causal):
    """f32 tensors with head_dim 64 / 128 run on tensor cores with three TF32 products per product: same 1e-5 bar
    as the f32 GEMM, against the f32 oracle and its f64-accumulating variant; ragged last query and key tiles."""
    capi = pkg.capi
    q = util.gen_normal(capi, (b, hq, s, d), 441)
    k = util.gen_normal(capi, (b, hkv, s, d), 442)
    v = util.gen_normal(capi, (b, hkv, s, d), 443)
    o = run_attention(dev, capi, q, k, v, capi.F32, causal)
    assert np.isfinite(o).all()
    m = oracle.compare(o, oracle.attention_f32(q, k, v, causal))
    assert m["rel_max"] <= 1e-5 and m["rel_fro"] <= 1e-5, m


@pytest.mark.parametrize("b,hq,hkv,s,d,causal", [(1, 4, 2, 300, 64, True), (2, 2, 2, 129, 96, False), (1, 2, 1, 1000, 32, True),
                                                    (1, 8, 2, 2048, 64, True)])
def test_attention_bf16_small_head_dims(dev, pkg, oracle, b, hq, hkv, s, d, causal):
    """16-bit data with head_dim 32 / 64 / 96: the warp-level tensor-core kernel (the inputs are TF32 numbers, so
    Q K^T is one product and P V two)."""
    capi = pkg.capi
    q, k, v = bf16_qkv(capi, b, hq, hkv, s, d, seed=471)
    o = run_attention(dev, capi, q, k, v, capi.BF16, causal).view(np.uint16)
    ref32, _ = oracle.attention_bf16(q, k, v, causal)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)


def test_attention_f16_head_dim_64(dev, pkg, oracle):
    capi = pkg.capi
    qf, kf, vf = (util.gen_normal(capi, (1, 2, 200, 64), 480 + i) for i in range(3))
    qh, kh, vh = (util.f32_to_f16_bits(t) for t in (qf, kf, vf))
    oh = run_attention(dev, capi, qh, kh, vh, capi.F16, True).view(np.float16).astype(np.float32)
    ref = oracle.attention_f32(*(t.view(np.float16).astype(np.float32) for t in (qh, kh, vh)), True)
    util.assert_16bit_close(oracle, oh, ref)


def test_attention_f32_other_head_dim_fp32_pipe(dev, pkg, oracle):
    capi = pkg.capi
    b, hq, hkv, s, d = 1, 2, 1, 70, 80  # head_dim 80 on f32 data: the FP32-pipe kernel
    q = util.gen_normal(capi, (b, hq, s, d), 451)
    k = util.gen_normal(capi, (b, hkv, s, d), 452)
    v = util.gen_normal(capi, (b, hkv, s, d), 453)
    o = run_attention(dev, capi, q, k, v, capi.F32, True)
    m = oracle.compare(o, oracle.attention_f32(q, k, v, True))
    assert m["rel_max"] <= 1e-5 and m["rel_fro"] <= 1e-5, m


def test_attention_f32_large_scores(dev, pkg, oracle):
    """Scores of a few hundred: the running maximum and the rescaling of the accumulator matter."""
    capi = pkg.capi
    q = 6.0 * util.gen_normal(capi, (1, 2, 500, 128), 461)
    k = util.gen_normal(capi, (1, 2, 500, 128), 462)
    v = util.gen_normal(capi, (1, 2, 500, 128), 463)
    o = run_attention(dev, capi, q, k, v, capi.F32, False)
    m = oracle.compare(o, oracle.attention_f32(q, k, v, False))
    assert m["rel_max"] <= 2e-5 and m["rel_fro"] <= 1e-5, m


def test_attention_f16_and_other_head_dim(dev, pkg, oracle):
    capi = pkg.capi
    b, h, s, d = 1, 2, 96, 80  # head_dim 80: FP32-pipe kernel on 16-bit data
    q, k, v = bf16_qkv(capi, b, h, h, s, d, seed=421)
    o = run_attention(dev, capi, q, k, v, capi.BF16, True).view(np.uint16)
    ref32, _ = oracle.attention_bf16(q, k, v, True)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)
    # f16 inputs on the tensor-core kernel
    qf, kf, vf = (util.gen_normal(capi, (1, 2, 256, 128), 430 + i) for i in range(3))
    qh, kh, vh = (util.f32_to_f16_bits(t) for t in (qf, kf, vf))
    oh = run_attention(dev, capi, qh, kh, vh, capi.F16, False).view(np.float16).astype(np.float32)
    ref = oracle.attention_f32(*(t.view(np.float16).astype(np.float32) for t in (qh, kh, vh)), False)
    util.assert_16bit_close(oracle, oh, ref)


def test_attention_bad_args(dev, pkg):
    capi = pkg.capi
    t = torch.zeros(1024, dtype=torch.int16, device="cuda:0")
    p = t.data_ptr()
    dev.attention(capi.BF16, 0, 1, 1, 128, 128, p, p, p, p)  # empty batch: no-op
    with pytest.raises(pkg.hal.KernelError):
        dev.attention(capi.BF16, 1, 3, 2, 128, 128, p, p, p, p)  # heads_q not a multiple of heads_kv
    with pytest.raises(pkg.hal.KernelError):
        dev.attention(capi.BF16, 1, 1, 1, 128, 512, p, p, p, p)  # head_dim too large


@pytest.mark.parametrize("causal", [False, True])
def test_attention_long_sequence_sampled_rows(dev, pkg, oracle, causal):
    """seq 4096 (the attention configuration's length): sampled query rows per head against the oracle."""
    capi = pkg.capi
    b, hq, hkv, s, d = 1, 4, 4, 4096, 128
    q, k, v = bf16_qkv(capi, b, hq, hkv, s, d)
    o = run_attention(dev, capi, q, k, v, capi.BF16, causal).view(np.uint16)
    for row0 in (0, 1920, 4032):
        ref32, _ = oracle.attention_bf16(q, k, v, causal, q_row0=row0, q_rows=64)
        util.assert_16bit_close(oracle, oracle.bf16_to_f32(np.ascontiguousarray(o[:, :, row0:row0 + 64])), ref32, row0)


def test_attention_gqa_16k_sampled_rows(dev, pkg, oracle):
    """One KV group of the 16384-long grouped-query configuration (8 query heads, causal)."""
    capi = pkg.capi
    b, hq, hkv, s, d = 1, 8, 1, 16384, 128
    q, k, v = bf16_qkv(capi, b, hq, hkv, s, d, seed=501)
    o = run_attention(dev, capi, q, k, v, capi.BF16, True).view(np.uint16)
    for row0 in (0, 8128, 16320):
        ref32, _ = oracle.attention_bf16(q, k, v, True, q_row0=row0, q_rows=64)
        util.assert_16bit_close(oracle, oracle.bf16_to_f32(np.ascontiguousarray(o[:, :, row0:row0 + 64])), ref32, row0)


def test_attention_host_path(dev, pkg, oracle):
    capi = pkg.capi
    b, hq, hkv, s, d = 2, 4, 2, 512, 128
    q, k, v = bf16_qkv(capi, b, hq, hkv, s, d, seed=441)
    o = np.zeros_like(q)
    dev.attention_host(capi.BF16, b, hq, hkv, s, d, q.ctypes.data, k.ctypes.data, v.ctypes.data, o.ctypes.data,
                       causal=True)
    ref32, _ = oracle.attention_bf16(q, k, v, True)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)


def _sampled_heads_check(dev, pkg, oracle, batch, hq, hkv, seq, causal, heads, what):
    """Runs the full configuration on device-generated bf16 N(0,1) data (per-head scales as the GQA configuration
    has them) and checks sampled (batch, head) x query-row blocks against the oracle: the head and batch indexing
    of the timed launches, which small cases cannot reach."""
    capi = pkg.capi
    g = torch.Generator(device="cuda:0").manual_seed(401)
    mk = lambda h: torch.randn(batch, h, seq, 128, device="cuda:0", generator=g)
    q, k, v = mk(hq), mk(hkv), mk(hkv)
    if hq != hkv:  # one scale per query head and per KV head, uniform in [0.5, 2)
        q *= (torch.rand(1, hq, 1, 1, device="cuda:0", generator=g) * 1.5 + 0.5)
        skv = torch.rand(1, hkv, 1, 1, device="cuda:0", generator=g) * 1.5 + 0.5
        k *= skv
        v *= skv
    q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
    o = torch.full_like(q, float("nan"))
    dev.attention(capi.BF16, batch, hq, hkv, seq, 128, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                  causal=causal, stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    assert not torch.isnan(o.float()).any()
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    group = hq // hkv
    over = 0
    for (b, h) in heads:
        qh, kh, vh = bits(q[b, h][None, None]), bits(k[b, h // group][None, None]), bits(v[b, h // group][None, None])
        for row0 in (0, seq // 2 - 32, seq - 64):
            ref32, _ = oracle.attention_bf16(qh, kh, vh, causal, q_row0=row0, q_rows=64)
            got = oracle.bf16_to_f32(bits(o[b, h, row0:row0 + 64][None, None]))
            m = util.assert_16bit_close(oracle, got, ref32, (what, b, h, row0))
            over += m["over_2e-2"]
    print(f"[parity] {what}: {len(heads)} heads x 3 row blocks, elements over 2e-2: {over}")


@pytest.mark.parametrize("causal", [False, True])
def test_attention_b8_h32_s4096_head_indexing(dev, pkg, oracle, causal):
    _sampled_heads_check(dev, pkg, oracle, 8, 32, 32, 4096, causal, [(0, 0), (0, 31), (3, 17), (7, 31)],
                         f"b8 h32 s4096 causal={causal}")


def test_attention_gqa_b2_64_8_s16384_head_indexing(dev, pkg, oracle):
    _sampled_heads_check(dev, pkg, oracle, 2, 64, 8, 16384, True, [(0, 0), (0, 63), (1, 9), (1, 56)], "gqa b2 64/8 s16384")


def test_attention_causal_launch_order_ragged_last_band(dev, pkg, oracle):
    """The causal launch order walks bands of KV heads whose K and V fit the L2 together; at seq 16384 a band is
    4 KV heads, so 6 heads leave a last band of 2 (MHA) and 3 KV heads of a 6/3 GQA a single short one."""
    _sampled_heads_check(dev, pkg, oracle, 1, 6, 6, 16384, True, [(0, 0), (0, 3), (0, 4), (0, 5)], "b1 h6 s16384")
    _sampled_heads_check(dev, pkg, oracle, 3, 2, 1, 16384, True, [(0, 1), (1, 0), (2, 1)], "gqa b3 2/1 s16384")
