"""Writes tests/golden/*.npz: small seeded cases with float64 numpy results.

The reference ships no numeric vectors for matmul / softmax / attention / the row operators (its tests
assert emitted text), and none of its code can run here, so these vectors pin the
C++ oracle against an independent float64 statement of the same linalg semantics
(oracle/oracle_np.py) and against drift of the input generator.  Regenerate with
    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import __graft_entry__ as entry  # noqa: E402
import util  # noqa: E402
from oracle import oracle_np as onp  # noqa: E402


def main() -> None:
    capi = entry.load_package().capi
    out = Path(__file__).resolve().parent
    # generator: first elements of each stream kind
    np.savez(out / "generator.npz",
             uniform_101=util.gen_uniform(capi, (64,), 101),
             normal_201=util.gen_normal(capi, (64,), 201, 3.0),
             normal_201_from_1000=util.gen_normal(capi, (16,), 201, 3.0, first=1000),
             outliers_202=util.plant_outliers(capi, np.zeros(2000, np.float32), 202).nonzero()[0].astype(np.int64))
    # softmax
    x = util.softmax_input(capi, 6, 96)
    np.savez(out / "softmax.npz", x=x, y=onp.softmax(x))
    # gemm f32 and bf16
    a, b = util.gen_uniform(capi, (24, 40), 101), util.gen_uniform(capi, (40, 16), 102)
    ab, bb = util.to_bf16(capi, a), util.to_bf16(capi, b)
    np.savez(out / "gemm.npz", a=a, b=b, c=onp.gemm(a, b), c_t=onp.gemm(a, np.ascontiguousarray(b.T), True),
             a_bf16=ab, b_bf16=bb, c_bf16=onp.gemm(onp.bf16_bits_to_f32(ab), onp.bf16_bits_to_f32(bb)))
    # attention: plain, causal, grouped
    q = util.gen_normal(capi, (2, 4, 24, 16), 401)
    k = util.gen_normal(capi, (2, 2, 24, 16), 402)
    v = util.gen_normal(capi, (2, 2, 24, 16), 403)
    np.savez(out / "attention.npz", q=q, k=k, v=v, o_gqa_causal=onp.attention(q, k, v, True),
             o_gqa_full=onp.attention(q, k, v, False),
             o_mha_full=onp.attention(q[:, :2], k, v, False), o_mha_causal=onp.attention(q[:, :2], k, v, True))
    # the other row operators: rms_norm, row sum / max, silu * mul
    xr = util.gen_normal(capi, (6, 96), 601, 3.0)
    gate, up = util.gen_normal(capi, (6, 96), 602, 4.0), util.gen_normal(capi, (6, 96), 603)
    np.savez(out / "rowops.npz", x=xr, eps=np.float32(1e-5), rms=onp.rms_norm(xr, 1e-5), row_sum=onp.reduce(xr, "sum"),
             row_max=onp.reduce(xr, "max"), gate=gate, up=up, silu=onp.silu_mul(gate), silu_mul=onp.silu_mul(gate, up))
    # decode attention: one query token per head against a partly filled, grouped KV cache
    qd = util.gen_normal(capi, (2, 4, 16), 801)
    kd, vd = util.gen_normal(capi, (2, 2, 24, 16), 802), util.gen_normal(capi, (2, 2, 24, 16), 803)
    np.savez(out / "attention_decode.npz", q=qd, k_cache=kd, v_cache=vd, seq_len=np.int64(19), o=onp.attention_decode(qd, kd, vd, 19))
    print("wrote", sorted(p.name for p in out.glob("*.npz")))


if __name__ == "__main__":
    main()
