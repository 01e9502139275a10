"""Independent float64 numpy statement of the same operators, for small cases.

Used to cross-check the C++ oracle (which is what the CUDA kernels are compared
with).  TEST INFRASTRUCTURE ONLY.  Each function cites the reference lines whose
semantics it states.
"""
from __future__ import annotations

import numpy as np


def bf16_bits_to_f32(x: np.ndarray) -> np.ndarray:
    """arith.extf (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1249-1303)."""
    return (x.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """arith.truncf, round-to-nearest-even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def gemm(a: np.ndarray, b: np.ndarray, b_transposed: bool = False) -> np.ndarray:
    """linalg.fill 0 + linalg.matmul (mlir_to_linalg.rs:1345-1393), in float64."""
    b64 = b.astype(np.float64)
    return a.astype(np.float64) @ (b64.T if b_transposed else b64)


def softmax(x: np.ndarray) -> np.ndarray:
    """linalg.softmax dimension(1) (mlir_to_linalg.rs:1305-1343), in float64."""
    x = x.astype(np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def rms_norm(x: np.ndarray, eps: float) -> np.ndarray:
    """x * rsqrt(mean(x^2) + eps) per row (mlir_to_linalg.rs:1666-1767), in float64."""
    x = x.astype(np.float64)
    return x / np.sqrt((x * x).sum(axis=1, keepdims=True) / x.shape[1] + np.float64(np.float32(eps)))


def reduce(x: np.ndarray, kind: str) -> np.ndarray:
    """Row sums or row maxima (mlir_to_linalg.rs:545-550), in float64."""
    x = x.astype(np.float64)
    return x.max(axis=1) if kind == "max" else x.sum(axis=1)


def silu_mul(gate: np.ndarray, up=None) -> np.ndarray:
    """silu(gate) [* up], silu(x) = x / (1 + exp(-x)) (mlir_to_linalg.rs:774-782, :425), in float64."""
    g = gate.astype(np.float64)
    with np.errstate(over="ignore"):
        s = g / (1.0 + np.exp(-g))
    return s if up is None else s * up.astype(np.float64)


# Element-wise operators in float64, as the linalg bridge defines them (mlir_to_linalg.rs:422-470 named
# linalg ops; :756-790 rsqrt / sigmoid / silu / relu; :805-905 scale; :907-982 clamp = min(max(x, lo), hi)).
EWISE = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
    "max": np.maximum, "min": np.minimum,
    "exp": np.exp, "log": np.log, "neg": lambda a: -a, "tanh": np.tanh, "abs": np.abs, "sqrt": np.sqrt,
    "rsqrt": lambda a: 1.0 / np.sqrt(a), "sigmoid": lambda a: 1.0 / (1.0 + np.exp(-a)),
    "silu": lambda a: a / (1.0 + np.exp(-a)), "relu": lambda a: np.maximum(a, 0.0),
    "scale": lambda a, c: a * np.float64(np.float32(c)),
    "clamp": lambda a, lo, hi: np.minimum(np.maximum(a, np.float64(np.float32(lo))), np.float64(np.float32(hi))),
}


def rope(x: np.ndarray, start_pos: int, theta: float) -> np.ndarray:
    """Rotary embedding of x [batch, seq_len, heads, d] (mlir_to_msl.rs:10883-10908), in float64."""
    x = x.astype(np.float64)
    b, s, h, d = x.shape
    i = np.arange(d // 2, dtype=np.float64)
    ang = (start_pos + np.arange(s, dtype=np.float64))[:, None] / np.float64(np.float32(theta)) ** (2.0 * i / d)[None, :]
    c, sn = np.cos(ang)[None, :, None, :], np.sin(ang)[None, :, None, :]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * sn
    out[..., 1::2] = x0 * sn + x1 * c
    return out


def attention_decode(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, seq_len: int) -> np.ndarray:
    """One query token per head against the first seq_len cache positions (mlir_to_msl.rs:10747-10812), in float64.
    q: [batch, hq, d]; caches: [batch, hkv, max_seq, d]."""
    q, k, v = q.astype(np.float64), k_cache.astype(np.float64)[:, :, :seq_len], v_cache.astype(np.float64)[:, :, :seq_len]
    b, hq, d = q.shape
    group = hq // k.shape[1]
    k, v = np.repeat(k, group, axis=1), np.repeat(v, group, axis=1)
    s = np.einsum("bhd,bhpd->bhp", q, k) / np.sqrt(d)
    s = np.exp(s - s.max(axis=2, keepdims=True))
    return np.einsum("bhp,bhpd->bhd", s / s.sum(axis=2, keepdims=True), v)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool) -> np.ndarray:
    """transpose, matmul, scale 1/sqrt(D), [causal mask col > row -> -inf], softmax, matmul
    (mlir_to_linalg.rs:1781-1902, :1191-1244); grouped KV heads with
    kv_head = h // (hq // hkv) (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1657-1673).
    q: [batch, hq, s, d]; k, v: [batch, hkv, s, d]."""
    q, k, v = (t.astype(np.float64) for t in (q, k, v))
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = np.empty_like(q)
    scale = 1.0 / np.sqrt(float(d))
    for bi in range(b):
        for h in range(hq):
            g = h // group
            sc = (q[bi, h] @ k[bi, g].T) * scale
            if causal:
                sc = np.where(np.triu(np.ones((s, s), bool), 1), -np.inf, sc)
            out[bi, h] = softmax(sc) @ v[bi, g]
    return out
