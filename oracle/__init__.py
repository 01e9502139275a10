"""CPU oracle for the tile_std matmul / row-softmax / fused-attention hot path.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline / reference legs of ``bench.py``; never by the product package.

PARITY UNPINNED: the reference holds no numeric golden vectors for these
operators and its linalg CPU executor is not in its tree, so the C++ restatement
(``oracle.cpp``, bound here through ctypes) is cross-checked only against the
independent float64 numpy statement in ``oracle_np``.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "_build" / "liboracle.so"
_LIB = None

_i64, _vp = C.c_int64, C.c_void_p


def build(force: bool = False) -> Path:
    """Compiles oracle.cpp with the Makefile beside it (g++ -O3 -fopenmp)."""
    src = _DIR / "oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        h = C.CDLL(str(build()))
        h.orc_num_threads.restype = C.c_int
        h.orc_set_num_threads.argtypes = [C.c_int]
        h.orc_set_num_threads.restype = None
        h.orc_gemm_f32.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, C.c_int]
        h.orc_gemm_f64acc.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, C.c_int]
        h.orc_gemm_bf16.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, C.c_int]
        h.orc_softmax_f32.argtypes = [_vp, _vp, _i64, _i64]
        h.orc_softmax_f64acc.argtypes = [_vp, _vp, _i64, _i64]
        h.orc_softmax_bf16.argtypes = [_vp, _vp, _vp, _i64, _i64]
        h.orc_attention_f32.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, C.c_int]
        h.orc_attention_bf16.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, C.c_int, _i64, _i64]
        h.orc_rms_norm_f32.argtypes = [_vp, _vp, _i64, _i64, C.c_float, C.c_int]
        h.orc_rms_norm_bf16.argtypes = [_vp, _vp, _vp, _i64, _i64, C.c_float]
        h.orc_reduce_f32.argtypes = [_vp, _vp, _i64, _i64, C.c_int, C.c_int]
        h.orc_silu_mul_f32.argtypes = [_vp, _vp, _vp, _i64, C.c_int]
        h.orc_silu_mul_bf16.argtypes = [_vp, _vp, _vp, _vp, _i64]
        h.orc_attention_decode_f32.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]
        h.orc_attention_decode_bf16.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64]
        h.orc_rope_f32.argtypes = [_vp, _i64, _i64, _i64, _i64, _i64, C.c_float, C.c_int]
        h.orc_kv_cache_update.argtypes = [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64]
        h.orc_attention_prefill_f32.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]
        h.orc_compare_f32.argtypes = [_vp, _vp, _i64, C.c_double, _vp]
        h.orc_bf16_to_f32.argtypes = [_vp, _vp, _i64]
        h.orc_f32_to_bf16.argtypes = [_vp, _vp, _i64]
        for name in ("orc_gemm_f32", "orc_gemm_f64acc", "orc_gemm_bf16", "orc_softmax_f32", "orc_softmax_f64acc",
                     "orc_softmax_bf16", "orc_attention_f32", "orc_attention_bf16", "orc_compare_f32",
                     "orc_bf16_to_f32", "orc_f32_to_bf16", "orc_rms_norm_f32", "orc_rms_norm_bf16", "orc_reduce_f32",
                     "orc_silu_mul_f32", "orc_silu_mul_bf16", "orc_attention_decode_f32", "orc_attention_decode_bf16", "orc_rope_f32", "orc_kv_cache_update", "orc_attention_prefill_f32"):
            getattr(h, name).restype = None
        _LIB = h
    return _LIB


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> int:
    """Sets the OpenMP thread count of the calling thread's parallel regions; returns what is then in force."""
    lib().orc_set_num_threads(int(n))
    return num_threads()


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x), _p(out), x.size)
    return out


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), x.size)
    return out


def gemm_f32(a: np.ndarray, b: np.ndarray, b_transposed: bool = False, f64_acc: bool = False) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    c = np.empty((m, n), np.float32)
    fn = lib().orc_gemm_f64acc if f64_acc else lib().orc_gemm_f32
    fn(_p(a), _p(b), _p(c), m, n, k, int(b_transposed))
    return c


def gemm_bf16(a: np.ndarray, b: np.ndarray, b_transposed: bool = False):
    """Returns (unrounded f32 result, RNE bf16 bit patterns)."""
    a = np.ascontiguousarray(a, np.uint16)
    b = np.ascontiguousarray(b, np.uint16)
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    c32 = np.empty((m, n), np.float32)
    c16 = np.empty((m, n), np.uint16)
    lib().orc_gemm_bf16(_p(a), _p(b), _p(c32), _p(c16), m, n, k, int(b_transposed))
    return c32, c16


def softmax_f32(x: np.ndarray, f64_acc: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    fn = lib().orc_softmax_f64acc if f64_acc else lib().orc_softmax_f32
    fn(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


def softmax_bf16(x: np.ndarray):
    """Returns (unrounded f32 result, RNE bf16 bit patterns)."""
    x = np.ascontiguousarray(x, np.uint16)
    y32 = np.empty(x.shape, np.float32)
    y16 = np.empty(x.shape, np.uint16)
    lib().orc_softmax_bf16(_p(x), _p(y32), _p(y16), x.shape[0], x.shape[1])
    return y32, y16


def rms_norm_f32(x: np.ndarray, eps: float, f64_acc: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_rms_norm_f32(_p(x), _p(y), x.shape[0], x.shape[1], eps, int(f64_acc))
    return y


def rms_norm_bf16(x: np.ndarray, eps: float):
    """Returns (unrounded f32 result, RNE bf16 bit patterns)."""
    x = np.ascontiguousarray(x, np.uint16)
    y32 = np.empty(x.shape, np.float32)
    y16 = np.empty(x.shape, np.uint16)
    lib().orc_rms_norm_bf16(_p(x), _p(y32), _p(y16), x.shape[0], x.shape[1], eps)
    return y32, y16


def reduce_f32(x: np.ndarray, kind: str, f64_acc: bool = False) -> np.ndarray:
    """Row sums ('sum') or row maxima ('max') of a [rows, cols] f32 matrix -> [rows]."""
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape[0], np.float32)
    lib().orc_reduce_f32(_p(x), _p(y), x.shape[0], x.shape[1], int(kind == "max"), int(f64_acc))
    return y


def silu_mul_f32(gate: np.ndarray, up, f64_acc: bool = False) -> np.ndarray:
    gate = np.ascontiguousarray(gate, np.float32)
    y = np.empty_like(gate)
    upc = None if up is None else np.ascontiguousarray(up, np.float32)
    lib().orc_silu_mul_f32(_p(gate), None if upc is None else _p(upc), _p(y), gate.size, int(f64_acc))
    return y


def silu_mul_bf16(gate: np.ndarray, up):
    """Returns (unrounded f32 result, RNE bf16 bit patterns)."""
    gate = np.ascontiguousarray(gate, np.uint16)
    upc = None if up is None else np.ascontiguousarray(up, np.uint16)
    y32 = np.empty(gate.shape, np.float32)
    y16 = np.empty(gate.shape, np.uint16)
    lib().orc_silu_mul_bf16(_p(gate), None if upc is None else _p(upc), _p(y32), _p(y16), gate.size)
    return y32, y16


def rope_f32(x: np.ndarray, start_pos: int, theta: float, f64_acc: bool = False) -> np.ndarray:
    """x: [batch, seq_len, heads, d]; returns the rotated copy."""
    y = np.array(x, np.float32, order="C", copy=True)
    b, s, h, d = y.shape
    lib().orc_rope_f32(_p(y), b, s, h, d, start_pos, theta, int(f64_acc))
    return y


def kv_cache_update(src: np.ndarray, cache: np.ndarray, start_pos: int) -> np.ndarray:
    """src: [batch, seq_len, heads, d]; cache: [batch, heads, max_seq, d] (same dtype); returns the updated copy."""
    src = np.ascontiguousarray(src)
    out = np.array(cache, order="C", copy=True)
    assert src.dtype == out.dtype
    b, s, h, d = src.shape
    lib().orc_kv_cache_update(_p(src), _p(out), src.dtype.itemsize, b, s, h, d, start_pos, out.shape[2])
    return out


def attention_prefill_f32(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, start_pos: int, f64_acc: bool = False) -> np.ndarray:
    """q: [seq_len, hq, d] (token-major); caches: [hkv, max_seq, d]; token s sees positions 0 .. start_pos + s."""
    q = np.ascontiguousarray(q, np.float32)
    k_cache = np.ascontiguousarray(k_cache, np.float32)
    v_cache = np.ascontiguousarray(v_cache, np.float32)
    s, hq, d = q.shape
    hkv, max_seq, _ = k_cache.shape
    o = np.empty_like(q)
    lib().orc_attention_prefill_f32(_p(q), _p(k_cache), _p(v_cache), _p(o), hq, hkv, s, start_pos, max_seq, d, int(f64_acc))
    return o


def attention_decode_f32(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, seq_len: int, f64_acc: bool = False) -> np.ndarray:
    """q: [batch, hq, d]; caches: [batch, hkv, max_seq, d]; positions < seq_len take part."""
    q = np.ascontiguousarray(q, np.float32)
    k_cache = np.ascontiguousarray(k_cache, np.float32)
    v_cache = np.ascontiguousarray(v_cache, np.float32)
    b, hq, d = q.shape
    _, hkv, max_seq, _ = k_cache.shape
    o = np.empty_like(q)
    lib().orc_attention_decode_f32(_p(q), _p(k_cache), _p(v_cache), _p(o), b, hq, hkv, seq_len, max_seq, d, int(f64_acc))
    return o


def attention_decode_bf16(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, seq_len: int):
    """bf16 bit patterns in; returns (unrounded f32 result, RNE bf16 bit patterns)."""
    q = np.ascontiguousarray(q, np.uint16)
    k_cache = np.ascontiguousarray(k_cache, np.uint16)
    v_cache = np.ascontiguousarray(v_cache, np.uint16)
    b, hq, d = q.shape
    _, hkv, max_seq, _ = k_cache.shape
    o32 = np.empty(q.shape, np.float32)
    o16 = np.empty(q.shape, np.uint16)
    lib().orc_attention_decode_bf16(_p(q), _p(k_cache), _p(v_cache), _p(o32), _p(o16), b, hq, hkv, seq_len, max_seq, d)
    return o32, o16


def attention_f32(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool) -> np.ndarray:
    """q: [batch, hq, s, d]; k, v: [batch, hkv, s, d]."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    b, hq, s, d = q.shape
    o = np.empty_like(q)
    lib().orc_attention_f32(_p(q), _p(k), _p(v), _p(o), b, hq, k.shape[1], s, d, int(causal))
    return o


def attention_bf16(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool, q_row0: int = 0, q_rows: int = -1):
    """bf16 bit patterns in; returns (unrounded f32, RNE bf16) for query rows [q_row0, q_row0+q_rows)."""
    q = np.ascontiguousarray(q, np.uint16)
    k = np.ascontiguousarray(k, np.uint16)
    v = np.ascontiguousarray(v, np.uint16)
    b, hq, s, d = q.shape
    if q_rows < 0:
        q_rows = s - q_row0
    o32 = np.empty((b, hq, q_rows, d), np.float32)
    o16 = np.empty((b, hq, q_rows, d), np.uint16)
    lib().orc_attention_bf16(_p(q), _p(k), _p(v), _p(o32), _p(o16), b, hq, k.shape[1], s, d, int(causal), q_row0, q_rows)
    return o32, o16


def compare(y: np.ndarray, r: np.ndarray, floor_r: float = 0.0) -> dict:
    """Parity metrics of a result ``y`` against the oracle ``r`` (both f32)."""
    y = np.ascontiguousarray(y, np.float32)
    r = np.ascontiguousarray(r, np.float32)
    assert y.shape == r.shape
    out = np.zeros(5, np.float64)
    lib().orc_compare_f32(_p(y), _p(r), y.size, float(floor_r), _p(out))
    return {"max_abs": out[0], "max_ref": out[1], "rel_max": out[0] / out[1] if out[1] else out[0],
            "rel_fro": out[2] / out[3] if out[3] else out[2], "max_elem_rel": out[4]}
