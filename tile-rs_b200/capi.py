"""ctypes binding of ``include/tile_sm100.h``.

``lib()`` loads ``libtile_sm100.so`` from this directory (building it with nvcc
when it is missing or stale) and declares every prototype of the header, so a
wrong argument count or type fails in Python instead of corrupting a call.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

from . import build as _build

OK, ERR_INVALID, ERR_NO_DEVICE, ERR_MEMORY, ERR_LAUNCH = 0, 1, 2, 3, 4
ERR_STREAM, ERR_RUNTIME, ERR_TIMEOUT, ERR_BUFFER, ERR_EMIT = 5, 6, 7, 8, 9
F32, F16, BF16 = 0, 1, 2
DTYPE_SIZE = {F32: 4, F16: 2, BF16: 2}

c_i32, c_i64, c_u32, c_u64, c_sz, c_vp = C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_size_t, C.c_void_p


class SoftmaxDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("rows", c_i64), ("cols", c_i64)]


class GemmDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("out_dtype", c_i32), ("b_transposed", c_i32), ("batch", c_i32),
                ("m", c_i64), ("n", c_i64), ("k", c_i64), ("lda", c_i64), ("ldb", c_i64), ("ldc", c_i64)]


class RmsNormDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("rows", c_i64), ("cols", c_i64), ("eps", C.c_float)]


class ReduceDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("kind", c_i32), ("rows", c_i64), ("cols", c_i64)]


class SiluMulDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("rows", c_i64), ("cols", c_i64)]


REDUCE_SUM, REDUCE_MAX = 0, 1


class RopeDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("batch", c_i32), ("seq_len", c_i32), ("heads", c_i32), ("head_dim", c_i32),
                ("start_pos", c_i32), ("theta", C.c_float)]


class KvCacheUpdateDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("batch", c_i32), ("seq_len", c_i32), ("heads", c_i32), ("head_dim", c_i32),
                ("start_pos", c_i32), ("max_seq", c_i32)]


class AttentionPrefillDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("heads_q", c_i32), ("heads_kv", c_i32), ("seq_len", c_i32), ("start_pos", c_i32),
                ("max_seq", c_i32), ("head_dim", c_i32)]


class AttentionDecodeDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("batch", c_i32), ("heads_q", c_i32), ("heads_kv", c_i32), ("seq_len", c_i32),
                ("max_seq", c_i32), ("head_dim", c_i32)]


class AttentionDesc(C.Structure):
    _fields_ = [("dtype", c_i32), ("causal", c_i32), ("batch", c_i32), ("heads_q", c_i32),
                ("heads_kv", c_i32), ("seq", c_i32), ("head_dim", c_i32)]


OP_SOFTMAX, OP_GEMM, OP_ATTENTION = 0, 1, 2


class MultiJob(C.Structure):
    _fields_ = [("op", c_i32), ("desc", c_vp), ("inputs", c_vp * 3), ("out", c_vp), ("launches", c_i32),
                ("timeout_ms", c_i32)]


class MultiReport(C.Structure):
    _fields_ = [("ordinal", c_i32), ("status", c_i32), ("first", c_i64), ("count", c_i64), ("upload_ms", C.c_float),
                ("kernel_ms", C.c_float), ("download_ms", C.c_float), ("total_ms", C.c_float), ("device_status", c_u32),
                ("message", C.c_char * 160)]


P = C.POINTER
MULTI_WORKER_FN = C.CFUNCTYPE(c_i32, c_vp, P(MultiJob), c_i32, c_i64, c_i64, P(MultiReport))
# name -> (restype, argtypes); every symbol the header declares
PROTOTYPES = {
    "tsm100_version": (c_i32, []),
    "tsm100_last_error": (c_sz, [C.c_char_p, c_sz]),
    "tsm100_device_count": (c_i32, [P(c_i32)]),
    "tsm100_device_open": (c_i32, [c_i32, P(c_vp)]),
    "tsm100_device_close": (c_i32, [c_vp]),
    "tsm100_device_ordinal": (c_i32, [c_vp, P(c_i32)]),
    "tsm100_device_name": (c_i32, [c_vp, C.c_char_p, c_sz]),
    "tsm100_mem_info": (c_i32, [c_vp, P(c_sz), P(c_sz)]),
    "tsm100_device_sm_count": (c_i32, [c_vp, P(c_i32)]),
    "tsm100_device_status": (c_i32, [c_vp, c_vp, P(c_u32)]),
    "tsm100_selftest_wait_timeout": (c_i32, [c_vp, c_u32, P(c_u32), c_vp]),
    "tsm100_stream_create": (c_i32, [c_vp, P(c_vp)]),
    "tsm100_stream_destroy": (c_i32, [c_vp, c_vp]),
    "tsm100_stream_synchronize": (c_i32, [c_vp, c_vp]),
    "tsm100_stream_query": (c_i32, [c_vp, c_vp, P(c_i32)]),
    "tsm100_event_create": (c_i32, [c_vp, P(c_vp)]),
    "tsm100_event_record": (c_i32, [c_vp, c_vp, c_vp]),
    "tsm100_event_synchronize": (c_i32, [c_vp, c_vp]),
    "tsm100_event_elapsed_ms": (c_i32, [c_vp, c_vp, c_vp, P(C.c_float)]),
    "tsm100_event_destroy": (c_i32, [c_vp, c_vp]),
    "tsm100_alloc": (c_i32, [c_vp, c_sz, P(c_vp)]),
    "tsm100_free": (c_i32, [c_vp, c_vp]),
    "tsm100_host_alloc": (c_i32, [c_sz, P(c_vp)]),
    "tsm100_host_free": (c_i32, [c_vp]),
    "tsm100_memcpy_h2d": (c_i32, [c_vp, c_vp, c_vp, c_sz, c_vp]),
    "tsm100_memcpy_d2h": (c_i32, [c_vp, c_vp, c_vp, c_sz, c_vp]),
    "tsm100_memset": (c_i32, [c_vp, c_vp, c_i32, c_sz, c_vp]),
    "tsm100_module_load": (c_i32, [c_vp, C.c_char_p, P(c_vp)]),
    "tsm100_module_unload": (c_i32, [c_vp]),
    "tsm100_launch": (c_i32, [c_vp, C.c_char_p, c_u32, P(c_vp), c_u32, c_vp]),
    "tsm100_softmax": (c_i32, [c_vp, P(SoftmaxDesc), c_vp, c_vp, c_vp]),
    "tsm100_rms_norm": (c_i32, [c_vp, P(RmsNormDesc), c_vp, c_vp, c_vp]),
    "tsm100_reduce": (c_i32, [c_vp, P(ReduceDesc), c_vp, c_vp, c_vp]),
    "tsm100_silu_mul": (c_i32, [c_vp, P(SiluMulDesc), c_vp, c_vp, c_vp, c_vp]),
    "tsm100_gemm": (c_i32, [c_vp, P(GemmDesc), c_vp, c_vp, c_vp, c_vp]),
    "tsm100_gemm_static_scratch": (c_i32, [P(GemmDesc), c_vp, c_vp, c_vp, c_vp, P(c_u32)]),
    "tsm100_attention": (c_i32, [c_vp, P(AttentionDesc), c_vp, c_vp, c_vp, c_vp, c_vp]),
    "tsm100_rope": (c_i32, [c_vp, P(RopeDesc), c_vp, c_vp]),
    "tsm100_kv_cache_update": (c_i32, [c_vp, P(KvCacheUpdateDesc), c_vp, c_vp, c_vp]),
    "tsm100_attention_prefill": (c_i32, [c_vp, P(AttentionPrefillDesc), c_vp, c_vp, c_vp, c_vp, c_vp]),
    "tsm100_attention_decode": (c_i32, [c_vp, P(AttentionDecodeDesc), c_vp, c_vp, c_vp, c_vp, c_vp]),
    "tsm100_softmax_host": (c_i32, [c_vp, P(SoftmaxDesc), c_vp, c_vp]),
    "tsm100_gemm_host": (c_i32, [c_vp, P(GemmDesc), c_vp, c_vp, c_vp]),
    "tsm100_attention_host": (c_i32, [c_vp, P(AttentionDesc), c_vp, c_vp, c_vp, c_vp]),
    "tsm100_shard_range": (c_i32, [c_i64, c_i32, c_i32, P(c_i64), P(c_i64)]),
    "tsm100_multi_plan": (c_i32, [P(MultiJob), c_i32, c_i32, P(c_i64), P(c_i64)]),
    "tsm100_multi_run": (c_i32, [P(MultiJob), P(c_i32), c_i32, P(MultiReport)]),
    "tsm100_multi_run_with": (c_i32, [P(MultiJob), P(c_i32), c_i32, P(MultiReport), MULTI_WORKER_FN, c_vp]),
    "tsm100_multi_release": (c_i32, []),
    "tsm100_emit": (c_i32, [C.c_char_p, c_sz, C.c_char_p, c_sz, P(c_sz), C.c_char_p, c_sz, P(c_sz)]),
    "tsm100_emit_descriptors": (c_i32, [C.c_char_p, c_sz, C.c_char_p, c_sz, P(c_sz)]),
    "tsm100_target_name": (C.c_char_p, []),
    "tsm100_target_ext": (C.c_char_p, []),
    "tsm100_fill_uniform_f32": (c_i32, [c_vp, c_i64, c_u64, c_i64]),
    "tsm100_fill_normal_f32": (c_i32, [c_vp, c_i64, c_u64, c_i64, C.c_double]),
    "tsm100_fill_normal_bf16": (c_i32, [c_vp, c_i64, c_u64, c_i64, C.c_double, C.c_float]),
    "tsm100_plant_outliers_f32": (c_i32, [c_vp, c_i64, c_u64, c_i64, c_u32, C.c_float]),
    "tsm100_scale_f32": (c_i32, [c_vp, c_i64, C.c_float]),
    "tsm100_f32_to_bf16": (c_i32, [c_vp, c_vp, c_i64]),
    "tsm100_bf16_to_f32": (c_i32, [c_vp, c_vp, c_i64]),
}

_LIB: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """The loaded library, with prototypes declared. Raises if it cannot be built or loaded."""
    global _LIB
    if _LIB is None:
        path = _build.build_library()
        handle = C.CDLL(str(path))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError names the missing export
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    lib().tsm100_last_error(buf, len(buf))
    return buf.value.decode(errors="replace")
