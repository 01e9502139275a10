"""Host-side mirror of the reference's ``tile_hal`` crate over the C ABI.

Same names, argument meaning and error behaviour as the Rust traits, so a test
written against ``tile_hal`` reads the same here:

* ``HalError`` + variants        crates/tile_hal/src/error.rs:5-35
* ``BackendKind`` / ``BackendSelector``  crates/tile_hal/src/backend.rs:5-113
* ``Device`` (``CudaSm100Device``)       crates/tile_hal/src/device.rs:25-57, cuda.rs:293-417
* ``Stream``                             crates/tile_hal/src/stream.rs:7-10, cuda.rs:134-166
* ``DeviceBuffer``                       crates/tile_hal/src/buffer.rs:32-55, cuda.rs:170-218
* ``KernelLauncher`` / ``LaunchGrid``    crates/tile_hal/src/kernel.rs:23-79, cuda.rs:222-289

What differs from the reference's CUDA backend, on purpose: copies are ordered
on the stream they are given (the reference ignores it), several devices can be
open in one process, kernels are looked up once per module, and events time
work on the device.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import capi


# ---- errors (error.rs:5-35) -------------------------------------------------
class HalError(Exception):
    kind = "runtime error"

    def __str__(self) -> str:  # Display impl, error.rs:21-32
        return f"{self.kind}: {self.args[0] if self.args else ''}"


class DeviceError(HalError):
    kind = "device error"


class MemoryError_(HalError):
    kind = "memory error"


class KernelError(HalError):
    kind = "kernel error"


class StreamError(HalError):
    kind = "stream error"


class BackendNotAvailable(HalError):
    kind = "backend not available"


class RuntimeError_(HalError):
    kind = "runtime error"


_CODE_TO_ERROR = {
    capi.ERR_INVALID: KernelError, capi.ERR_NO_DEVICE: BackendNotAvailable, capi.ERR_MEMORY: MemoryError_,
    capi.ERR_LAUNCH: KernelError, capi.ERR_STREAM: StreamError, capi.ERR_RUNTIME: RuntimeError_,
    capi.ERR_TIMEOUT: RuntimeError_, capi.ERR_BUFFER: RuntimeError_, capi.ERR_EMIT: KernelError,
}


def check(status: int) -> None:
    """Raises the HalError variant the status code maps to (check_cu, cuda.rs:124-130)."""
    if status != capi.OK:
        raise _CODE_TO_ERROR.get(status, RuntimeError_)(capi.last_error())


# ---- backend selection (backend.rs:5-113) ----------------------------------
class BackendKind(enum.Enum):
    Ascend = "cpp"
    Cuda = "gpu"
    Musa = "musa"
    Aie = "aie"
    Nki = "nki"
    Spirv = "spirv"
    Msl = "msl"
    Bang = "bang"
    Gaudi = "gaudi"

    @staticmethod
    def from_codegen_path(s: str) -> Optional["BackendKind"]:
        """backend.rs:28-41, with the one added arm ``"cuda_sm100" -> Cuda``."""
        table = {"cpp": BackendKind.Ascend, "pto": BackendKind.Ascend, "gpu": BackendKind.Cuda,
                 "cuda_sm100": BackendKind.Cuda, "musa": BackendKind.Musa, "aie": BackendKind.Aie,
                 "nki": BackendKind.Nki, "spirv": BackendKind.Spirv, "msl": BackendKind.Msl,
                 "bang": BackendKind.Bang, "gaudi": BackendKind.Gaudi}
        return table.get(s)

    def codegen_path(self) -> str:
        return self.value


class BackendSelector:
    def __init__(self, kind: BackendKind):
        self._kind = kind

    @staticmethod
    def from_env() -> "BackendSelector":
        """TILERS_CODEGEN_PATH, then ACLRS_CODEGEN_PATH, default "cpp" (backend.rs:70-78)."""
        path = os.environ.get("TILERS_CODEGEN_PATH") or os.environ.get("ACLRS_CODEGEN_PATH") or "cpp"
        kind = BackendKind.from_codegen_path(path)
        if kind is None:
            raise BackendNotAvailable(f"unknown codegen path: {path}")
        return BackendSelector(kind)

    def kind(self) -> BackendKind:
        return self._kind

    def device(self, ordinal: int) -> "CudaSm100Device":
        if self._kind is not BackendKind.Cuda:
            raise BackendNotAvailable(f"{self._kind.name} backend not compiled (enable the feature flag)")
        return CudaSm100Device(ordinal)


# ---- kernel launch shapes (kernel.rs:9-79) ---------------------------------
class KernelMode(enum.Enum):
    Vector = 0
    Matrix = 1
    General = 2


@dataclass(frozen=True)
class LaunchGrid:
    blocks: int
    threads_per_block: int = 1
    shared_mem_bytes: int = 0

    @staticmethod
    def blocks_(n: int) -> "LaunchGrid":  # LaunchGrid::blocks
        return LaunchGrid(n, 1, 0)

    @staticmethod
    def cuda(blocks: int, threads: int) -> "LaunchGrid":
        return LaunchGrid(blocks, threads, 0)

    def with_shared_mem(self, nbytes: int) -> "LaunchGrid":
        return LaunchGrid(self.blocks, self.threads_per_block, nbytes)


@dataclass(frozen=True)
class MemInfo:  # device.rs:9-15
    free: int
    total: int


# ---- stream / event ---------------------------------------------------------
class Stream:
    def __init__(self, device: "CudaSm100Device"):
        self._dev = device
        h = C.c_void_p()
        check(capi.lib().tsm100_stream_create(device._h, C.byref(h)))
        self._h = h

    @property
    def raw(self) -> int:
        return self._h.value or 0

    def synchronize(self) -> None:
        check(capi.lib().tsm100_stream_synchronize(self._dev._h, self._h))

    def query(self) -> bool:
        done = C.c_int32()
        check(capi.lib().tsm100_stream_query(self._dev._h, self._h, C.byref(done)))
        return bool(done.value)

    def close(self) -> None:
        if self._h is not None:
            capi.lib().tsm100_stream_destroy(self._dev._h, self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Event:
    def __init__(self, device: "CudaSm100Device"):
        self._dev = device
        h = C.c_void_p()
        check(capi.lib().tsm100_event_create(device._h, C.byref(h)))
        self._h = h

    def record(self, stream: Optional[Stream]) -> None:
        check(capi.lib().tsm100_event_record(self._dev._h, self._h, stream._h if stream else None))

    def synchronize(self) -> None:
        check(capi.lib().tsm100_event_synchronize(self._dev._h, self._h))

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float()
        check(capi.lib().tsm100_event_elapsed_ms(self._dev._h, self._h, later._h, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            if self._h is not None:
                capi.lib().tsm100_event_destroy(self._dev._h, self._h)
                self._h = None
        except Exception:
            pass


# ---- buffers (buffer.rs:32-55) ----------------------------------------------
class DeviceBuffer:
    """``count`` elements of ``dtype`` (a numpy dtype) in device memory; freed on drop."""

    def __init__(self, device: "CudaSm100Device", count: int, dtype) -> None:
        self._dev = device
        self.dtype = np.dtype(dtype)
        self._count = int(count)
        p = C.c_void_p()
        check(capi.lib().tsm100_alloc(device._h, self._count * self.dtype.itemsize, C.byref(p)))
        self._p = p

    def len(self) -> int:
        return self._count

    def __len__(self) -> int:
        return self._count

    def is_empty(self) -> bool:
        return self._count == 0

    def as_raw_ptr(self) -> int:
        return self._p.value or 0

    as_raw_mut_ptr = as_raw_ptr

    def copy_from_host(self, host: np.ndarray, stream: Optional[Stream]) -> None:
        host = np.ascontiguousarray(host)
        if host.size != self._count or host.dtype.itemsize != self.dtype.itemsize:
            raise MemoryError_(f"host slice has {host.size} elements, buffer has {self._count}")
        check(capi.lib().tsm100_memcpy_h2d(self._dev._h, self._p, host.ctypes.data, host.nbytes,
                                           stream._h if stream else None))
        # pageable host memory: the call has already consumed `host`
        if stream is not None:
            stream.synchronize()

    def copy_to_host(self, stream: Optional[Stream]) -> np.ndarray:
        out = np.empty(self._count, dtype=self.dtype)
        check(capi.lib().tsm100_memcpy_d2h(self._dev._h, out.ctypes.data, self._p, out.nbytes,
                                           stream._h if stream else None))
        if stream is not None:
            stream.synchronize()
        else:
            check(capi.lib().tsm100_stream_synchronize(self._dev._h, None))
        return out

    def free(self) -> None:
        if self._p is not None and self._p.value:
            capi.lib().tsm100_free(self._dev._h, self._p)
        self._p = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


# ---- launcher (kernel.rs:23-42) ---------------------------------------------
class KernelLauncher:
    def __init__(self, device: "CudaSm100Device"):
        self._dev = device
        self._modules: list = []

    def load(self, path, mode: KernelMode = KernelMode.Vector) -> None:
        m = C.c_void_p()
        check(capi.lib().tsm100_module_load(self._dev._h, os.fsencode(str(path)), C.byref(m)))
        self._modules.append(m)

    def launch(self, name: str, grid: LaunchGrid, args: Sequence[int], stream: Optional[Stream]) -> None:
        """``args``: raw device pointers in the kernel's declaration order (kernel.rs:32-34)."""
        if not self._modules:
            raise KernelError("no kernel binary loaded")
        arr = (C.c_void_p * len(args))(*[C.c_void_p(int(a)) for a in args])
        last = None
        for m in reversed(self._modules):
            st = capi.lib().tsm100_launch(m, name.encode(), grid.blocks, arr, len(args), stream._h if stream else None)
            if st == capi.OK:
                return
            last = st
            if "not found in module" not in capi.last_error():
                break
        check(last)

    def launch_described(self, kernel, grid: LaunchGrid, buffers: Sequence["DeviceBuffer"], stream: Optional[Stream]) -> None:
        """Launch with the kernel's TileKernel descriptor (codegen.TileKernel): the three uses
        kernel.rs:163-168 names - the argument count, and every buffer's size against
        ``grid.blocks`` per-block tiles, are checked before anything reaches the device."""
        if len(buffers) != len(kernel.args):
            raise KernelError(f"{kernel.name} takes {len(kernel.args)} buffers ({kernel.num_inputs} in, "
                              f"{kernel.num_outputs} out), got {len(buffers)}")
        for a, b in zip(kernel.args, buffers):
            need = a.bytes_for(grid.blocks)
            have = b.len() * b.dtype.itemsize
            if have < need:
                raise KernelError(f"{kernel.name}: buffer {a.index} ({a.role}, {a.dtype}) holds {have} bytes, "
                                  f"{grid.blocks} blocks need {need}")
        ptrs = [b.as_raw_mut_ptr() if a.role == "output" else b.as_raw_ptr() for a, b in zip(kernel.args, buffers)]
        self.launch(kernel.name, grid, ptrs, stream)

    def __del__(self):
        try:
            for m in self._modules:
                capi.lib().tsm100_module_unload(m)
            self._modules = []
        except Exception:
            pass


# ---- device (device.rs:25-57) -------------------------------------------------
class CudaSm100Device:
    def __init__(self, ordinal: int):
        h = C.c_void_p()
        check(capi.lib().tsm100_device_open(int(ordinal), C.byref(h)))
        self._h = h
        buf = C.create_string_buffer(256)
        check(capi.lib().tsm100_device_name(h, buf, len(buf)))
        self._name = buf.value.decode()
        self._ordinal = int(ordinal)

    @staticmethod
    def device_count() -> int:
        n = C.c_int32()
        check(capi.lib().tsm100_device_count(C.byref(n)))
        return n.value

    def ordinal(self) -> int:
        return self._ordinal

    def name(self) -> str:
        return self._name

    def sm_count(self) -> int:
        n = C.c_int32()
        check(capi.lib().tsm100_device_sm_count(self._h, C.byref(n)))
        return n.value

    def create_stream(self) -> Stream:
        return Stream(self)

    def create_event(self) -> Event:
        return Event(self)

    def alloc(self, count: int, dtype=np.float32) -> DeviceBuffer:
        return DeviceBuffer(self, count, dtype)

    def alloc_f32(self, count: int) -> DeviceBuffer:  # DynDevice::alloc_f32, backend.rs:118-125
        return DeviceBuffer(self, count, np.float32)

    def alloc_from_slice(self, data: np.ndarray, stream: Optional[Stream]) -> DeviceBuffer:
        data = np.ascontiguousarray(data)
        buf = DeviceBuffer(self, data.size, data.dtype)
        buf.copy_from_host(data.reshape(-1), stream)
        return buf

    def mem_info(self) -> MemInfo:
        f, t = C.c_size_t(), C.c_size_t()
        check(capi.lib().tsm100_mem_info(self._h, C.byref(f), C.byref(t)))
        return MemInfo(f.value, t.value)

    def create_launcher(self) -> KernelLauncher:
        return KernelLauncher(self)

    def status(self, stream: Optional[Stream] = None) -> int:
        v = C.c_uint32()
        check(capi.lib().tsm100_device_status(self._h, stream._h if stream else None, C.byref(v)))
        return v.value

    # -- typed operators (device pointers as ints) --
    def softmax(self, dtype: int, rows: int, cols: int, x: int, y: int, stream: int = 0) -> None:
        d = capi.SoftmaxDesc(dtype, rows, cols)
        check(capi.lib().tsm100_softmax(self._h, C.byref(d), x, y, stream or None))

    def rms_norm(self, dtype: int, rows: int, cols: int, eps: float, x: int, y: int, stream: int = 0) -> None:
        d = capi.RmsNormDesc(dtype, rows, cols, eps)
        check(capi.lib().tsm100_rms_norm(self._h, C.byref(d), x, y, stream or None))

    def reduce(self, dtype: int, kind: int, rows: int, cols: int, x: int, y: int, stream: int = 0) -> None:
        """Row sums (capi.REDUCE_SUM) or maxima (capi.REDUCE_MAX) of a rows x cols tile into y[rows]."""
        d = capi.ReduceDesc(dtype, kind, rows, cols)
        check(capi.lib().tsm100_reduce(self._h, C.byref(d), x, y, stream or None))

    def silu_mul(self, dtype: int, rows: int, cols: int, gate: int, up: Optional[int], y: int, stream: int = 0) -> None:
        """y = silu(gate) * up; up=None gives silu(gate)."""
        d = capi.SiluMulDesc(dtype, rows, cols)
        check(capi.lib().tsm100_silu_mul(self._h, C.byref(d), gate, up or None, y, stream or None))

    def gemm(self, dtype: int, m: int, n: int, k: int, a: int, b: int, c: int, *, out_dtype: Optional[int] = None,
             b_transposed: bool = False, batch: int = 1, lda: int = 0, ldb: int = 0, ldc: int = 0, stream: int = 0) -> None:
        """C = A * B; lda / ldb / ldc are row pitches in elements (0: packed rows)."""
        d = capi.GemmDesc(dtype, dtype if out_dtype is None else out_dtype, int(b_transposed), batch, m, n, k, lda, ldb, ldc)
        check(capi.lib().tsm100_gemm(self._h, C.byref(d), a, b, c, stream or None))

    def attention(self, dtype: int, batch: int, heads_q: int, heads_kv: int, seq: int, head_dim: int, q: int, k: int,
                  v: int, o: int, *, causal: bool = False, stream: int = 0) -> None:
        d = capi.AttentionDesc(dtype, int(causal), batch, heads_q, heads_kv, seq, head_dim)
        check(capi.lib().tsm100_attention(self._h, C.byref(d), q, k, v, o, stream or None))

    def rope(self, dtype: int, batch: int, seq_len: int, heads: int, head_dim: int, start_pos: int, theta: float, x: int,
             stream: int = 0) -> None:
        """In-place rotary embedding of x [batch, seq_len, heads, head_dim] at positions start_pos .. start_pos + seq_len - 1."""
        d = capi.RopeDesc(dtype, batch, seq_len, heads, head_dim, start_pos, theta)
        check(capi.lib().tsm100_rope(self._h, C.byref(d), x, stream or None))

    def kv_cache_update(self, dtype: int, batch: int, seq_len: int, heads: int, head_dim: int, start_pos: int, max_seq: int,
                        src: int, cache: int, stream: int = 0) -> None:
        """cache[b, h, start_pos + s] = src[b, s, h] for src [batch, seq_len, heads, d], cache [batch, heads, max_seq, d]."""
        d = capi.KvCacheUpdateDesc(dtype, batch, seq_len, heads, head_dim, start_pos, max_seq)
        check(capi.lib().tsm100_kv_cache_update(self._h, C.byref(d), src, cache, stream or None))

    def attention_prefill(self, dtype: int, heads_q: int, heads_kv: int, seq_len: int, start_pos: int, max_seq: int, head_dim: int,
                          q: int, k_cache: int, v_cache: int, o: int, stream: int = 0) -> None:
        """Causal attention of seq_len new tokens (token-major q, o) against the first start_pos + seq_len cache positions."""
        d = capi.AttentionPrefillDesc(dtype, heads_q, heads_kv, seq_len, start_pos, max_seq, head_dim)
        check(capi.lib().tsm100_attention_prefill(self._h, C.byref(d), q, k_cache, v_cache, o, stream or None))

    def attention_decode(self, dtype: int, batch: int, heads_q: int, heads_kv: int, seq_len: int, max_seq: int, head_dim: int,
                         q: int, k_cache: int, v_cache: int, o: int, stream: int = 0) -> None:
        """One query token per head against the first ``seq_len`` positions of a [batch, heads_kv, max_seq, d] cache."""
        d = capi.AttentionDecodeDesc(dtype, batch, heads_q, heads_kv, seq_len, max_seq, head_dim)
        check(capi.lib().tsm100_attention_decode(self._h, C.byref(d), q, k_cache, v_cache, o, stream or None))

    # -- operators on host buffers (upload + compute + download) --
    def softmax_host(self, dtype: int, rows: int, cols: int, x: int, y: int) -> None:
        d = capi.SoftmaxDesc(dtype, rows, cols)
        check(capi.lib().tsm100_softmax_host(self._h, C.byref(d), x, y))

    def gemm_host(self, dtype: int, m: int, n: int, k: int, a: int, b: int, c: int, *, out_dtype: Optional[int] = None,
                  b_transposed: bool = False, batch: int = 1, lda: int = 0, ldb: int = 0, ldc: int = 0) -> None:
        """The same on host buffers; the pitches describe the HOST matrices (device copies are packed)."""
        d = capi.GemmDesc(dtype, dtype if out_dtype is None else out_dtype, int(b_transposed), batch, m, n, k, lda, ldb, ldc)
        check(capi.lib().tsm100_gemm_host(self._h, C.byref(d), a, b, c))

    def attention_host(self, dtype: int, batch: int, heads_q: int, heads_kv: int, seq: int, head_dim: int, q: int,
                       k: int, v: int, o: int, *, causal: bool = False) -> None:
        d = capi.AttentionDesc(dtype, int(causal), batch, heads_q, heads_kv, seq, head_dim)
        check(capi.lib().tsm100_attention_host(self._h, C.byref(d), q, k, v, o))

    def close(self) -> None:
        if self._h is not None:
            capi.lib().tsm100_device_close(self._h)
            self._h = None
