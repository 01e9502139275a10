#!/usr/bin/env python
"""Benchmark of the tile-rs hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input that is already
resident in HBM.  The headline workload is the row softmax configuration (65536 x 4096
f32, 3*N(0,1) with 1 % of the entries at +20); every other configuration (bf16 softmax,
f32 and bf16 GEMMs, attention forward) is measured after it, each with its own sampled
check against the CPU oracle, CPU baseline, end-to-end (host buffers) figure and, on
several GPUs, strong-scaling figure.  Details go under "workloads", the figures of the
tensor-bound configurations once more, compactly, under "summary" at the end of the line.

Inputs are generated once on the host (counter-based generator of the library, the seeds and
laws of each configuration), uploaded, and read by the oracle from the same host buffers.
Under torchrun (N > 1) every rank carries the one-GPU configuration (weak scaling, the
reported value) and then its shard of that configuration (strong scaling: rows, batches,
N-column blocks, KV groups), the two in alternating blocks of steps for the strong-scaling
ratio; there is no collective on the data path.  Times are CUDA-event times on the launching
stream, maximum over ranks.

--impl reference times the CPU restatement of the reference's linalg semantics (the
oracle) on all host cores for the same configurations, each step a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

SOFTMAX_ROWS, SOFTMAX_COLS = 65536, 4096
HEAD_DIM = 128


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_threads(world: int = 1) -> int:
    """This process's share of the host cores (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    n = max(1, n // max(1, world))
    os.environ["OMP_NUM_THREADS"] = str(n)
    return n


# --------------------------------------------------------------------------- configurations
# name -> the configuration as both arms report it (identical dictionaries, so the two lines can be compared)
def catalogue_configs():
    l2_big = "inputs larger than L2 (no flush needed)"
    return {
        "softmax_f32": {"rows": SOFTMAX_ROWS, "cols": SOFTMAX_COLS, "law": "3*N(0,1), 1% of entries = +20, seeds 201/202", "l2": l2_big},
        "softmax_bf16": {"rows": SOFTMAX_ROWS, "cols": SOFTMAX_COLS, "law": "RNE(3*N(0,1), 1% of entries = +20), seeds 201/202", "l2": l2_big},
        "gemm_f32_512": {"m": 512, "n": 512, "k": 512, "problems": 1, "law": "uniform[-1,1), seeds 101/102", "l2": "inputs fit in L2 (3 MiB): a latency-bound configuration, timed back to back"},
        "gemm_f32_4096": {"m": 4096, "n": 4096, "k": 4096, "problems": 1, "law": "uniform[-1,1), seeds 101/102", "l2": l2_big},
        "gemm_bf16_8192": {"m": 8192, "n": 8192, "k": 8192, "problems": 1, "law": "N(0, sigma = K^-1/4), seeds 301/302", "l2": l2_big},
        "gemm_bf16_batched_4096": {"m": 4096, "n": 4096, "k": 4096, "problems": 64, "law": "N(0, sigma = K^-1/4), seeds 310+2b / 311+2b", "l2": l2_big},
        "attention_noncausal": {"batch": 8, "heads_q": 32, "heads_kv": 32, "seq": 4096, "head_dim": 128, "causal": False, "law": "N(0,1), seeds 401/402/403", "l2": l2_big},
        "attention_causal": {"batch": 8, "heads_q": 32, "heads_kv": 32, "seq": 4096, "head_dim": 128, "causal": True, "law": "N(0,1), seeds 401/402/403", "l2": l2_big},
        "attention_gqa_causal": {"batch": 2, "heads_q": 64, "heads_kv": 8, "seq": 16384, "head_dim": 128, "causal": True,
                                 "law": "N(0,1) seeds 501/502/503, one scale per query head and per KV head uniform[0.5,2) seed 504", "l2": l2_big},
        "attention_f32_causal": {"batch": 1, "heads_q": 32, "heads_kv": 32, "seq": 4096, "head_dim": 128, "causal": True, "law": "N(0,1), seeds 401/402/403, f32", "l2": l2_big},
        "rms_norm_f32": {"rows": SOFTMAX_ROWS, "cols": SOFTMAX_COLS, "law": "3*N(0,1) (device generator)", "l2": l2_big},
        "reduce_sum_f32": {"rows": SOFTMAX_ROWS, "cols": SOFTMAX_COLS, "law": "3*N(0,1) (device generator)", "l2": l2_big},
        "silu_mul_f32": {"rows": SOFTMAX_ROWS, "cols": SOFTMAX_COLS, "law": "N(0,1) (device generator)", "l2": l2_big},
        "silu_mul_bf16": {"rows": SOFTMAX_ROWS, "cols": SOFTMAX_COLS, "law": "N(0,1) (device generator)", "l2": l2_big},
        "attention_decode_bf16": {"kv_caches": 256, "q_heads_per_kv_head": 8, "seq_len": 16384, "head_dim": 128, "law": "N(0,1) (device generator)", "l2": l2_big},
    }


# the order workloads are measured and printed in: the tensor-bound configurations last
ORDER = ["softmax_f32", "softmax_bf16", "rms_norm_f32", "reduce_sum_f32", "silu_mul_f32", "silu_mul_bf16", "attention_decode_bf16",
         "attention_f32_causal", "gemm_f32_512", "gemm_f32_4096", "gemm_bf16_batched_4096", "attention_noncausal", "attention_gqa_causal",
         "attention_causal", "gemm_bf16_8192"]
SUMMARY = ["gemm_f32_512", "gemm_bf16_batched_4096", "attention_noncausal", "attention_gqa_causal", "attention_causal", "gemm_bf16_8192"]
METRIC = "row softmax HBM GB/s (GEMM / attention TFLOP/s under 'workloads' and 'summary')"


def config_for(name: str, reduced_units: int = 0) -> dict:
    cfg = {"workload": name + (" (REDUCED: --units)" if reduced_units else ""), **catalogue_configs()[name],
           "sharding": "independent units split over GPUs, no collective on the data path"}
    return cfg


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons while the timed region runs: NVML read
    calls every 5 ms from a thread of this process (the device is found by its UUID, so CUDA_VISIBLE_DEVICES
    does not matter); `nvidia-smi -lms 20` as a child process where the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    BITS = [0x8, 0x40, 0x20, 0x4]  # nvmlClocksEventReason: HwSlowdown, HwThermalSlowdown, SwThermalSlowdown, SwPowerCap

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread, self.stop, self.source = index, [], None, None, False, "none"

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(_torch().cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def __enter__(self):
        try:
            nv, h = self._nvml_handle()
            mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self.stop:
                    try:
                        mask = int(reasons(h))
                        self.rows.append([float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), mx] +
                                         ["Active" if mask & b else "Not Active" for b in self.BITS])
                    except Exception:
                        pass
                    time.sleep(0.005)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            self.source = "nvml"
            return self
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            self.source = "nvidia-smi"
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread:
            self.stop = True
            self.thread.join(timeout=1)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in list(self.rows):
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(self.NAMES, r[2:6]):
                if str(v).lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": self.source}


def _torch():
    import torch
    return torch


# --------------------------------------------------------------------------- host buffers
class HostBuf:
    """A page-locked host array from the library's allocator (copies from it run asynchronously)."""

    def __init__(self, ctx, shape, dtype):
        self.ctx, self.shape, self.dtype = ctx, tuple(shape), np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        self.ptr = C.c_void_p()
        ctx.hal.check(ctx.lib.tsm100_host_alloc(max(self.nbytes, 1), C.byref(self.ptr)))
        ct = {2: C.c_uint16, 4: C.c_float}[self.dtype.itemsize]
        self.array = np.ctypeslib.as_array(C.cast(self.ptr, C.POINTER(ct)), shape=(int(np.prod(self.shape)),)).reshape(self.shape)
        if self.dtype.itemsize == 2:
            self.array = self.array.view(np.uint16)

    @property
    def addr(self) -> int:
        return self.ptr.value

    def free(self):
        if self.ptr:
            self.array = None
            self.ctx.lib.tsm100_host_free(self.ptr)
            self.ptr = None


def fill_normal(ctx, buf: HostBuf, seed, sigma=1.0, first=0, factor=1.0, view=None):
    """N(0, sigma^2) * factor from the library's counter-based stream into a host buffer (or a slice of one)."""
    arr = buf.array if view is None else view
    n = arr.size
    if arr.dtype == np.uint16:
        ctx.hal.check(ctx.lib.tsm100_fill_normal_bf16(arr.ctypes.data, n, seed, first, float(sigma), float(factor)))
    else:
        ctx.hal.check(ctx.lib.tsm100_fill_normal_f32(arr.ctypes.data, n, seed, first, float(sigma)))
        if factor != 1.0:
            ctx.hal.check(ctx.lib.tsm100_scale_f32(arr.ctypes.data, n, float(factor)))


def upload(ctx, host: HostBuf):
    torch = _torch()
    tdt = torch.int16 if host.dtype.itemsize == 2 else torch.float32
    t = torch.empty(host.shape, dtype=tdt, device=ctx.tdev)
    ctx.hal.check(ctx.lib.tsm100_memcpy_h2d(ctx.dev._h, t.data_ptr(), host.ptr, host.nbytes, None))
    torch.cuda.synchronize()
    return t


def dev_rows_to_host(t, index):
    """Rows `index` (a list) of the first dimension of a device tensor, as a numpy array (16-bit as uint16)."""
    torch = _torch()
    sel = t[torch.tensor(list(index), device=t.device)].cpu().numpy()
    return sel.view(np.uint16) if sel.dtype == np.int16 else sel


def parity_16bit(oracle, got_f32, ref_f32):
    """The 16-bit bar: relative Frobenius <= 1e-2; |y - r| <= max(2e-2, half a bf16 ulp of |r| + 2^-9 |r|)."""
    m = oracle.compare(got_f32, ref_f32)
    ref = np.abs(np.asarray(ref_f32, np.float64))
    err = np.abs(np.asarray(got_f32, np.float64) - np.asarray(ref_f32, np.float64))
    tol = np.maximum(2e-2, 2.0 ** (np.floor(np.log2(np.maximum(ref, 1e-30))) - 8) + 2.0 ** -9 * ref)
    ok = bool(m["rel_fro"] <= 1e-2 and (err <= tol).all())
    return {"ok": ok, "max_abs": float(m["max_abs"]), "rel_fro": float(m["rel_fro"]), "over_2e-2": int((err > 2e-2).sum()),
            "elements": int(err.size), "tolerance": "rel_fro <= 1e-2, |y-r| <= max(2e-2, half a bf16 ulp of |r| + 2^-9 |r|) vs the unrounded f32 oracle"}


def parity_f32(oracle, got, ref):
    m = oracle.compare(got, ref)
    ok = bool(m["rel_max"] <= 1e-5 and m["rel_fro"] <= 1e-5)
    return {"ok": ok, "rel_max": float(m["rel_max"]), "rel_fro": float(m["rel_fro"]), "elements": int(np.asarray(got).size),
            "tolerance": "max|y-r|/max|r| <= 1e-5 and rel_fro <= 1e-5 vs the float64-accumulating oracle"}


# --------------------------------------------------------------------------- workloads
class Workload:
    """One configuration on one GPU.  `units` are what is sharded over GPUs; `work_per_unit` is the
    algorithmic bytes (HBM-bound) or flop (tensor-bound) of one unit."""
    name = ""
    bound = "hbm"          # or "tensor" / "tensor_f32"
    dtype = "f32"
    unit_name = "rows"
    strong_unit = None     # what a strong-scaling split deals out, if not `unit_name`
    launches_per_step = 1

    def __init__(self, ctx, units: int):
        self.ctx, self.units = ctx, units
        self.bufs = []

    def host(self, shape, dtype) -> HostBuf:
        b = HostBuf(self.ctx, shape, dtype)
        self.bufs.append(b)
        return b

    def work(self) -> float:
        return self.units * self.work_per_unit

    def strong_units(self) -> int:
        return self.units

    def step(self):
        self.step_range(0, self.strong_units())

    def free(self):
        for b in self.bufs:
            b.free()
        self.bufs = []


class SoftmaxWL(Workload):
    unit_name = "rows"

    def __init__(self, ctx, units, dtype="f32"):
        super().__init__(ctx, units)
        capi = ctx.pkg.capi
        self.dtype, self.cols, self.name = dtype, SOFTMAX_COLS, f"softmax_{dtype}"
        self.es = 4 if dtype == "f32" else 2
        self.code = capi.F32 if dtype == "f32" else capi.BF16
        self.work_per_unit = self.cols * self.es * 2  # one read + one write per element
        n = units * self.cols
        x32 = self.host((units, self.cols), np.float32)
        fill_normal(ctx, x32, 201, 3.0)
        ctx.hal.check(ctx.lib.tsm100_plant_outliers_f32(x32.ptr, n, 202, 0, 100, 20.0))
        if dtype == "f32":
            self.x_host = x32
        else:
            self.x_host = self.host((units, self.cols), np.uint16)
            ctx.hal.check(ctx.lib.tsm100_f32_to_bf16(x32.ptr, self.x_host.ptr, n))
            x32.free()
        self.x = upload(ctx, self.x_host)
        self.y = _torch().empty_like(self.x)
        self.y_host = None

    def step_range(self, first, count):
        off = first * self.cols * self.es
        self.ctx.dev.softmax(self.code, count, self.cols, self.x.data_ptr() + off, self.y.data_ptr() + off, stream=self.ctx.stream)

    def verify(self, oracle):
        rows = sorted({0, self.units // 3, self.units // 2, self.units - 1})
        xs, ys = self.x_host.array[rows], dev_rows_to_host(self.y, rows)
        if self.dtype == "f32":
            ref = oracle.softmax_f32(xs, f64_acc=True)
            v = parity_f32(oracle, ys, ref)
            v["ok"] = bool(v["ok"] and np.abs(ys.sum(axis=1) - 1).max() <= 1e-5)
        else:
            ref, _ = oracle.softmax_bf16(xs)
            v = parity_16bit(oracle, oracle.bf16_to_f32(ys), ref)
        v["rows"] = len(rows)
        return v

    def e2e_prepare(self):
        self.y_host = self.host((self.units, self.cols), self.x_host.dtype)
        return self.x_host.nbytes, self.y_host.nbytes, "tsm100_softmax_host (pinned host buffers, chunked copy/compute overlap)"

    def e2e_step(self):
        self.ctx.dev.softmax_host(self.code, self.units, self.cols, self.x_host.addr, self.y_host.addr)

    def e2e_check(self):
        rows = sorted({0, self.units // 2, self.units - 1})
        return bool(np.array_equal(self.y_host.array[rows], dev_rows_to_host(self.y, rows)))

    def cpu_run(self, oracle, seconds):
        rows = min(self.units, 4096)
        x = np.ascontiguousarray(self.x_host.array[:rows])
        fn = oracle.softmax_f32 if self.dtype == "f32" else oracle.softmax_bf16
        t0, done = time.perf_counter(), 0
        while True:
            fn(x)
            done += rows
            if time.perf_counter() - t0 >= seconds:
                break
        dt = time.perf_counter() - t0
        return done * self.work_per_unit / dt / 1e9, f"{rows} of {self.units} rows x {self.cols} cols, {done // rows} passes in {dt:.1f} s"


class RowOpWL(Workload):
    """rms_norm / row sum / silu * mul on the softmax configuration's shape (next-tier operators; device-generated input)."""
    unit_name = "rows"

    def __init__(self, ctx, units, op, dtype="f32"):
        super().__init__(ctx, units)
        torch, capi = _torch(), ctx.pkg.capi
        self.op, self.dtype, self.cols = op, dtype, SOFTMAX_COLS
        self.name = f"{op}_{dtype}"
        es = 4 if dtype == "f32" else 2
        self.code = capi.F32 if dtype == "f32" else capi.BF16
        tdt = torch.float32 if dtype == "f32" else torch.bfloat16
        g = torch.Generator(device=ctx.tdev).manual_seed(601)
        self.x = (torch.randn(units, self.cols, device=ctx.tdev, generator=g) * 3).to(tdt)
        streams = {"rms_norm": 2, "reduce_sum": 1, "silu_mul": 3}[op]
        self.work_per_unit = streams * self.cols * es + (es if op == "reduce_sum" else 0)
        self.y = torch.empty(units, device=ctx.tdev, dtype=tdt) if op == "reduce_sum" else torch.empty_like(self.x)
        self.up = torch.randn(units, self.cols, device=ctx.tdev, generator=g).to(tdt) if op == "silu_mul" else None

    def step_range(self, first, count):
        d, capi = self.ctx.dev, self.ctx.pkg.capi
        if self.op == "rms_norm":
            d.rms_norm(self.code, count, self.cols, 1e-5, self.x.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)
        elif self.op == "reduce_sum":
            d.reduce(self.code, capi.REDUCE_SUM, count, self.cols, self.x.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)
        else:
            d.silu_mul(self.code, count, self.cols, self.x.data_ptr(), self.up.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)


class GemmWL(Workload):
    bound, unit_name = "tensor", "problems"

    def __init__(self, ctx, units, m, n, k, dtype, name, seeds):
        super().__init__(ctx, units)
        capi = ctx.pkg.capi
        self.m, self.n, self.k, self.dtype, self.name = m, n, k, dtype, name
        self.work_per_unit = 2.0 * m * n * k
        self.single = units == 1 and catalogue_configs()[name]["problems"] == 1
        if self.single:
            self.strong_unit = "N columns"
        if dtype == "f32":
            self.bound, self.code, self.es, npdt = "tensor_f32", capi.F32, 4, np.float32
        else:
            self.code, self.es, npdt = capi.BF16, 2, np.uint16
        self.a_host, self.b_host = self.host((units, m, k), npdt), self.host((units, k, n), npdt)
        for b in range(units):
            sa, sb = seeds(b)
            if dtype == "f32":  # uniform[-1, 1)
                ctx.hal.check(ctx.lib.tsm100_fill_uniform_f32(self.a_host.array[b].ctypes.data, m * k, sa, 0))
                ctx.hal.check(ctx.lib.tsm100_fill_uniform_f32(self.b_host.array[b].ctypes.data, k * n, sb, 0))
            else:               # N(0, sigma^2) with variance 1/sqrt(K): outputs are O(1)
                fill_normal(ctx, None, sa, k ** -0.25, view=self.a_host.array[b])
                fill_normal(ctx, None, sb, k ** -0.25, view=self.b_host.array[b])
        self.a, self.b = upload(ctx, self.a_host), upload(ctx, self.b_host)
        self.c = _torch().empty((units, m, n), dtype=self.a.dtype, device=ctx.tdev)
        self.c_host = None

    def strong_units(self):
        return self.n if self.single else self.units

    def step(self):
        """The whole configuration through the C ABI with a descriptor built once (the 512^3 problem is latency-bound:
        building a ctypes structure per call costs as much as a tenth of its kernel)."""
        if not hasattr(self, "_desc"):
            capi = self.ctx.pkg.capi
            self._desc = capi.GemmDesc(self.code, self.code, 0, self.units, self.m, self.n, self.k, 0, 0, 0)
            self._call = (self.ctx.lib.tsm100_gemm, self.ctx.dev._h, C.byref(self._desc), self.a.data_ptr(), self.b.data_ptr(),
                          self.c.data_ptr(), self.ctx.stream or None)
        fn = self._call
        st = fn[0](*fn[1:])
        if st != 0:
            self.ctx.hal.check(st)

    def step_range(self, first, count):
        d, es = self.ctx.dev, self.es
        if self.single:  # columns [first, first + count) of C = A * B, in place inside the full matrices
            d.gemm(self.code, self.m, count, self.k, self.a.data_ptr(), self.b.data_ptr() + first * es, self.c.data_ptr() + first * es,
                   ldb=self.n, ldc=self.n, stream=self.ctx.stream)
        else:
            d.gemm(self.code, self.m, self.n, self.k, self.a.data_ptr() + first * self.m * self.k * es,
                   self.b.data_ptr() + first * self.k * self.n * es, self.c.data_ptr() + first * self.m * self.n * es,
                   batch=count, stream=self.ctx.stream)

    def _check_rows(self, oracle, c_rows, problem, rows, cols=None):
        a = np.ascontiguousarray(self.a_host.array[problem][rows])
        bm = self.b_host.array[problem]
        if cols is not None:
            bm = np.ascontiguousarray(bm[:, cols[0]:cols[1]])
        if self.dtype == "f32":
            return parity_f32(oracle, c_rows, oracle.gemm_f32(a, bm, f64_acc=True))
        ref32, _ = oracle.gemm_bf16(a, bm)
        return parity_16bit(oracle, oracle.bf16_to_f32(c_rows), ref32)

    def verify(self, oracle):
        problems = sorted({0, self.units // 2, self.units - 1})
        rows = sorted({0, self.m // 2 + 1, self.m - 1})
        out = None
        for p in problems:
            v = self._check_rows(oracle, dev_rows_to_host(self.c[p], rows), p, rows)
            if out is None:
                out = v
            else:
                out["ok"] = out["ok"] and v["ok"]
                for key in ("max_abs", "rel_fro", "rel_max"):
                    if key in v:
                        out[key] = max(out[key], v[key])
                for key in ("over_2e-2", "elements"):
                    if key in v:
                        out[key] += v[key]
        out["problems"], out["rows_per_problem"] = len(problems), len(rows)
        return out

    def verify_strong(self, oracle, first, count):
        """The N-column block this rank computes, written in place into a C full of sentinels."""
        if not self.single:
            return None
        torch = _torch()
        sentinel = 12345 if self.es == 2 else 777.0
        self.c.fill_(sentinel)
        self.step_range(first, count)
        torch.cuda.synchronize()
        rows = sorted({0, self.m // 2 + 1, self.m - 1})
        got = dev_rows_to_host(self.c[0], rows)
        v = self._check_rows(oracle, np.ascontiguousarray(got[:, first:first + count]), 0, rows, (first, first + count))
        outside = np.concatenate([got[:, :first].ravel(), got[:, first + count:].ravel()])
        v["ok"] = bool(v["ok"] and (outside == (np.uint16(sentinel) if self.es == 2 else np.float32(sentinel))).all())
        v["columns"] = [int(first), int(first + count)]
        self.step()  # the full result again, for the checks that follow
        torch.cuda.synchronize()
        return v

    def e2e_prepare(self):
        self.c_host = self.host((self.units, self.m, self.n), self.a_host.dtype)
        return self.a_host.nbytes + self.b_host.nbytes, self.c_host.nbytes, "tsm100_gemm_host (pinned host buffers; B resident, A and C streamed in row blocks; a batch one problem per stream slot)"

    def e2e_step(self):
        self.ctx.dev.gemm_host(self.code, self.m, self.n, self.k, self.a_host.addr, self.b_host.addr, self.c_host.addr, batch=self.units)

    def e2e_check(self):
        # The host-buffer call streams a large A in row blocks, each a launch of its own; the 16-bit pair kernel
        # orders its f32 sums by the waves of a launch, so a block may round a few results the other way: equal to
        # one 16-bit rounding step, and nearly all bits equal.  f32 results and single-block problems are bit-equal.
        rows = sorted({0, self.m // 2 + 1, self.m - 1})
        p = self.units - 1
        x, y = self.c_host.array[p][rows], dev_rows_to_host(self.c[p], rows)
        if np.array_equal(x, y):
            return True
        if self.dtype == "f32":
            return False
        xf, yf = self.ctx.oracle.bf16_to_f32(x), self.ctx.oracle.bf16_to_f32(y)
        step = np.maximum(np.abs(xf), np.abs(yf)) * np.float32(2.0 ** -7) + np.float32(1e-5)  # near zero: the f32 sums' own error (results are O(1))
        return bool((np.abs(xf - yf) <= step).all() and np.count_nonzero(x != y) <= 0.02 * x.size)

    def cpu_run(self, oracle, seconds):
        rows = min(self.m, 512 if self.dtype == "f32" and self.m <= 512 else 32)
        a = np.ascontiguousarray(self.a_host.array[0][:rows])
        bm = self.b_host.array[0]
        fn = (lambda: oracle.gemm_f32(a, bm)) if self.dtype == "f32" else (lambda: oracle.gemm_bf16(a, bm))
        t0, passes = time.perf_counter(), 0
        while True:
            fn()
            passes += 1
            if time.perf_counter() - t0 >= seconds:
                break
        dt = time.perf_counter() - t0
        flop = passes * 2.0 * rows * self.n * self.k
        what = "the whole problem" if rows == self.m else f"{rows} of {self.m} rows of C of one problem against the full B (cost is linear in rows)"
        return flop / dt / 1e12, f"{what}, {passes} passes in {dt:.1f} s"


class AttentionWL(Workload):
    bound, unit_name = "tensor", "kv_groups"

    def __init__(self, ctx, units, group, seq, causal, name, dtype="bf16", seeds=(401, 402, 403), head_scales=False, shared=None):
        super().__init__(ctx, units)
        capi = ctx.pkg.capi
        self.group, self.seq, self.causal, self.name, self.dtype = group, seq, causal, name, dtype
        if dtype == "f32":
            self.bound, self.code, self.es, npdt = "tensor_f32", capi.F32, 4, np.float32
        else:
            self.code, self.es, npdt = capi.BF16, 2, np.uint16
        self.work_per_unit = 4.0 * group * seq * seq * HEAD_DIM * (0.5 if causal else 1.0)
        if shared is not None:  # the non-causal and causal configurations read the same tensors
            self.q_host, self.k_host, self.v_host, self.q, self.k, self.v = shared
        else:
            self.q_host = self.host((units, group, seq, HEAD_DIM), npdt)
            self.k_host, self.v_host = self.host((units, 1, seq, HEAD_DIM), npdt), self.host((units, 1, seq, HEAD_DIM), npdt)
            cfg = catalogue_configs()[name]
            hkv = cfg["heads_kv"]
            if head_scales:  # one factor per query head and one per KV head, uniform[0.5, 2): seed 504, heads_q values then heads_kv
                u = np.empty(cfg["heads_q"] + hkv, np.float32)
                ctx.hal.check(ctx.lib.tsm100_fill_uniform_f32(u.ctypes.data, u.size, 504, 0))
                u = 1.25 + 0.75 * u
            head = seq * HEAD_DIM
            for unit in range(units):  # unit = (batch, KV head), batch-major; the streams are indexed as the full tensors are
                g = unit % hkv
                fq = float(1.0)
                for h in range(group):
                    if head_scales:
                        fq = float(u[g * group + h])
                    fill_normal(ctx, None, seeds[0], first=(unit * group + h) * head, factor=fq, view=self.q_host.array[unit, h])
                fkv = float(u[cfg["heads_q"] + g]) if head_scales else 1.0
                fill_normal(ctx, None, seeds[1], first=unit * head, factor=fkv, view=self.k_host.array[unit, 0])
                fill_normal(ctx, None, seeds[2], first=unit * head, factor=fkv, view=self.v_host.array[unit, 0])
            self.q, self.k, self.v = upload(ctx, self.q_host), upload(ctx, self.k_host), upload(ctx, self.v_host)
        self.o = _torch().empty_like(self.q)
        self.o_host = None

    def shared(self):
        return (self.q_host, self.k_host, self.v_host, self.q, self.k, self.v)

    def step_range(self, first, count):
        hq, hk = self.group * self.seq * HEAD_DIM * self.es, self.seq * HEAD_DIM * self.es
        self.ctx.dev.attention(self.code, count, self.group, 1, self.seq, HEAD_DIM, self.q.data_ptr() + first * hq,
                               self.k.data_ptr() + first * hk, self.v.data_ptr() + first * hk, self.o.data_ptr() + first * hq,
                               causal=self.causal, stream=self.ctx.stream)

    def verify(self, oracle):
        picks = sorted({(0, 0), (self.units // 2, self.group // 2), (self.units - 1, self.group - 1)})
        blocks = sorted({0, self.seq // 2 - 32, self.seq - 64})
        out, n = None, 0
        for (u, h) in picks:
            qh, kh, vh = self.q_host.array[u, h][None, None], self.k_host.array[u][None], self.v_host.array[u][None]
            o_head = self.o[u, h]
            if self.dtype == "f32":
                ref = oracle.attention_f32(qh, kh, vh, self.causal)[0, 0]
                v = parity_f32(oracle, o_head.cpu().numpy(), ref)
                n += 1
            else:
                v = None
                for row0 in blocks:
                    ref32, _ = oracle.attention_bf16(qh, kh, vh, self.causal, q_row0=row0, q_rows=64)
                    got = oracle.bf16_to_f32(o_head[row0:row0 + 64].cpu().numpy().view(np.uint16))
                    vb = parity_16bit(oracle, got, ref32[0, 0])
                    n += 1
                    if v is None:
                        v = vb
                    else:
                        v["ok"] = v["ok"] and vb["ok"]
                        v["max_abs"], v["rel_fro"] = max(v["max_abs"], vb["max_abs"]), max(v["rel_fro"], vb["rel_fro"])
                        v["over_2e-2"] += vb["over_2e-2"]
                        v["elements"] += vb["elements"]
            if out is None:
                out = v
            else:
                out["ok"] = out["ok"] and v["ok"]
                for key in ("max_abs", "rel_fro", "rel_max"):
                    if key in v:
                        out[key] = max(out[key], v[key])
                for key in ("over_2e-2", "elements"):
                    if key in v:
                        out[key] += v[key]
        out["heads"], out["row_blocks_checked"] = len(picks), n
        return out

    def e2e_prepare(self):
        self.o_host = self.host(self.q_host.shape, self.q_host.dtype)
        return self.q_host.nbytes + self.k_host.nbytes + self.v_host.nbytes, self.o_host.nbytes, "tsm100_attention_host (pinned host buffers, (batch, KV head) groups streamed in chunks)"

    def e2e_step(self):
        self.ctx.dev.attention_host(self.code, self.units, self.group, 1, self.seq, HEAD_DIM, self.q_host.addr, self.k_host.addr,
                                    self.v_host.addr, self.o_host.addr, causal=self.causal)

    def e2e_check(self):
        u, h = self.units - 1, self.group - 1
        return bool(np.array_equal(self.o_host.array[u, h, -64:], dev_rows_to_host(self.o[u, h], range(self.seq - 64, self.seq))))

    def cpu_run(self, oracle, seconds):
        """Whole query heads (every row of the head, so a causal head costs half a non-causal one), one after another."""
        t0, heads = time.perf_counter(), 0
        while True:
            u, h = heads % self.units, (heads // self.units) % self.group
            qh, kh, vh = self.q_host.array[u, h][None, None], self.k_host.array[u][None], self.v_host.array[u][None]
            if self.dtype == "f32":
                oracle.attention_f32(qh, kh, vh, self.causal)
            else:
                oracle.attention_bf16(qh, kh, vh, self.causal)
            heads += 1
            if time.perf_counter() - t0 >= seconds:
                break
        dt = time.perf_counter() - t0
        return heads * (self.work_per_unit / self.group) / dt / 1e12, f"{heads} of {self.units * self.group} query heads at full sequence length in {dt:.1f} s (cost is linear in heads)"

    def context(self):
        """torch's fused attention (a vendor kernel) on the same tensors: a yardstick printed beside the number, never on the product path."""
        torch = _torch()
        if self.dtype != "bf16":
            return None
        try:
            import torch.nn.functional as F
            q, k, v = (t.view(torch.bfloat16) for t in (self.q, self.k, self.v))
            kw = {"is_causal": self.causal}
            if self.group > 1:
                kw["enable_gqa"] = True
            for _ in range(2):
                F.scaled_dot_product_attention(q, k, v, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(5):
                F.scaled_dot_product_attention(q, k, v, **kw)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 5
            return {"torch_sdpa_tflops": round(self.work() / (ms * 1e-3) / 1e12, 1), "note": "vendor kernel through torch, same tensors, burst; context only"}
        except Exception as exc:  # a torch build without a fused kernel for this shape
            return {"torch_sdpa_tflops": None, "note": f"unavailable: {type(exc).__name__}"}


class DecodeWL(Workload):
    """One decode step: `units` (batch, KV head) caches of 16384 x 128 bf16, 8 query heads each (next-tier operator)."""
    unit_name, bound, dtype = "kv_caches", "hbm", "bf16"

    def __init__(self, ctx, units, seq=16384, group=8, name="attention_decode_bf16"):
        super().__init__(ctx, units)
        torch = _torch()
        self.seq, self.group, self.name = seq, group, name
        g = torch.Generator(device=ctx.tdev).manual_seed(801)
        self.q = torch.randn(units, group, HEAD_DIM, device=ctx.tdev, generator=g).to(torch.bfloat16)
        self.k = torch.randn(units, 1, seq, HEAD_DIM, device=ctx.tdev, generator=g).to(torch.bfloat16)
        self.v = torch.randn(units, 1, seq, HEAD_DIM, device=ctx.tdev, generator=g).to(torch.bfloat16)
        self.o = torch.empty_like(self.q)
        self.work_per_unit = 2.0 * seq * HEAD_DIM * 2 + 2.0 * group * HEAD_DIM * 2  # K and V once, q in, o out

    def step_range(self, first, count):
        self.ctx.dev.attention_decode(self.ctx.pkg.capi.BF16, count, self.group, 1, self.seq, self.seq, HEAD_DIM,
                                      self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.o.data_ptr(), stream=self.ctx.stream)


def make_workload(ctx, name, units=0, shared=None):
    """`units` > 0 overrides the configuration's size (a reduced case for profiler captures)."""
    cfg = catalogue_configs()[name]
    if name.startswith("softmax_"):
        return SoftmaxWL(ctx, units or cfg["rows"], name.split("_")[1])
    if name in ("rms_norm_f32", "reduce_sum_f32", "silu_mul_f32", "silu_mul_bf16"):
        op, dt = name.rsplit("_", 1)
        return RowOpWL(ctx, units or cfg["rows"], op, dt)
    if name == "attention_decode_bf16":
        return DecodeWL(ctx, units or cfg["kv_caches"])
    if name.startswith("gemm_"):
        dt = "f32" if "_f32_" in name else "bf16"
        if name == "gemm_bf16_batched_4096":
            seeds = lambda b: (310 + 2 * b, 311 + 2 * b)
        elif dt == "f32":
            seeds = lambda b: (101, 102)
        else:
            seeds = lambda b: (301, 302)
        return GemmWL(ctx, units or cfg["problems"], cfg["m"], cfg["n"], cfg["k"], dt, name, seeds)
    groups = cfg["batch"] * cfg["heads_kv"]
    gqa = name == "attention_gqa_causal"
    return AttentionWL(ctx, units or groups, cfg["heads_q"] // cfg["heads_kv"], cfg["seq"], cfg["causal"], name,
                       dtype="f32" if "_f32_" in name else "bf16", seeds=(501, 502, 503) if gqa else (401, 402, 403),
                       head_scales=gqa, shared=shared)


class Ctx:
    pass


def copy_probe(ctx, nbytes=1 << 30):
    """What the box gives plain page-locked copies, so that the end-to-end figure can be read against it: 1 GiB
    host-to-device alone, device-to-host alone, and both at once on two streams; every rank at the same time,
    slowest rank's time, aggregate GB/s per direction."""
    torch = _torch()
    h_in, h_out = HostBuf(ctx, (nbytes // 4,), np.float32), HostBuf(ctx, (nbytes // 4,), np.float32)
    d_in = torch.empty(nbytes // 4, dtype=torch.float32, device=ctx.tdev)
    d_out = torch.zeros(nbytes // 4, dtype=torch.float32, device=ctx.tdev)
    s1, s2 = ctx.dev.create_stream(), ctx.dev.create_stream()
    up = lambda: ctx.hal.check(ctx.lib.tsm100_memcpy_h2d(ctx.dev._h, d_in.data_ptr(), h_in.ptr, nbytes, s1.raw))
    down = lambda: ctx.hal.check(ctx.lib.tsm100_memcpy_d2h(ctx.dev._h, h_out.ptr, d_out.data_ptr(), nbytes, s2.raw))

    def timed(*fns):
        best = None
        for _ in range(3):
            torch.cuda.synchronize()
            if ctx.world > 1:
                ctx.dist.barrier()
            t0 = time.perf_counter()
            for fn in fns:
                fn()
            s1.synchronize()
            s2.synchronize()
            dt = max_over_ranks(ctx, time.perf_counter() - t0)
            best = dt if best is None else min(best, dt)
        return round(ctx.world * nbytes / best / 1e9, 1)

    out = {"bytes_each": nbytes, "h2d_alone_gbs": timed(up), "d2h_alone_gbs": timed(down), "both_gbs_per_direction": timed(up, down),
           "note": "aggregate over ranks, plain cudaMemcpyAsync of page-locked memory, best of 3"}
    h_in.free()
    h_out.free()
    return out


# --------------------------------------------------------------------------- timing
def time_steps(ctx, fn, steps, warmup):
    """Returns (total ms over `steps`, maximum over ranks; list of this rank's per-step ms), device-timed on the launching
    stream.  The total is taken between two events around the whole loop (an event after every step would add a few
    microseconds to each, a fifth of the 512^3 GEMM's own time); the per-step spread comes from a second, untimed pass."""
    torch = _torch()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    total = max_over_ranks(ctx, e0.elapsed_time(e1))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    assert ctx.dev.status() == 0, "a kernel reported a timed-out device-side wait"
    return total, per


def time_alternating(ctx, fn_a, fn_b, steps, warmup, block=5):
    """Times two loops against each other in the same thermal and power state: blocks of `block` steps of fn_a and of
    fn_b alternate, each block between two events.  Returns (ms per step of fn_a, of fn_b), each the maximum over ranks."""
    torch = _torch()
    for _ in range(warmup):
        fn_a()
        fn_b()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    torch.cuda.synchronize()
    rounds = max(1, (steps + block - 1) // block)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(2 * rounds + 1)]
    evs[0].record()
    for r in range(rounds):
        for _ in range(block):
            fn_a()
        evs[2 * r + 1].record()
        for _ in range(block):
            fn_b()
        evs[2 * r + 2].record()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    a = sum(evs[2 * r].elapsed_time(evs[2 * r + 1]) for r in range(rounds)) / (rounds * block)
    b = sum(evs[2 * r + 1].elapsed_time(evs[2 * r + 2]) for r in range(rounds)) / (rounds * block)
    assert ctx.dev.status() == 0, "a kernel reported a timed-out device-side wait"
    return max_over_ranks(ctx, a), max_over_ranks(ctx, b)


def max_over_ranks(ctx, value: float) -> float:
    if ctx.world == 1:
        return value
    t = _torch().tensor([value], device=ctx.tdev, dtype=_torch().float64)
    ctx.dist.all_reduce(t, op=ctx.dist.ReduceOp.MAX)
    return float(t.item())


def all_ranks_ok(ctx, ok: bool) -> bool:
    if ctx.world == 1:
        return ok
    t = _torch().tensor([0.0 if ok else 1.0], device=ctx.tdev, dtype=_torch().float64)
    ctx.dist.all_reduce(t, op=ctx.dist.ReduceOp.MAX)
    return float(t.item()) == 0.0


def roofline_for(wl, ms_per_launch, peaks):
    if wl.bound == "hbm":
        achieved, peak, unit, src = wl.work() / (ms_per_launch * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s", peaks["source"]
    elif wl.bound == "tensor":
        achieved, peak, unit, src = wl.work() / (ms_per_launch * 1e-3) / 1e12, peaks["bf16_tflops"], "TFLOP/s", peaks["source"]
    else:  # f32 operands: three TF32 products per product, and the TF32 rate is half the bf16 rate
        achieved, peak, unit = wl.work() / (ms_per_launch * 1e-3) / 1e12, peaks["bf16_tflops"] / 6.0, "TFLOP/s"
        src = peaks["source"] + " bf16 GEMM peak / 2 (TF32 rate) / 3 (products per f32-grade product)"
    return {"bound": "hbm" if wl.bound == "hbm" else "tensor", "achieved": round(achieved, 2), "peak": round(peak, 2), "unit": unit,
            "frac": round(achieved / peak, 4), "peak_source": src}


def sustained_run(ctx, wl, seconds, peaks, gpu_index):
    """The tensor-bound kernels draw the board's full power: the short timed run sees burst clocks, a loop of a
    second or more runs under the power cap.  Launches back to back for `seconds`, device-timed, clocks sampled;
    per-GPU throughput (the slowest rank's) against the measured sustained GEMM peak."""
    torch = _torch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    chunks = []
    with ClockSampler(gpu_index) as clk:
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < seconds:
            e0.record(torch.cuda.current_stream())
            for _ in range(20):
                wl.step()
            e1.record(torch.cuda.current_stream())
            e1.synchronize()
            chunks.append(e0.elapsed_time(e1) / 20)
    ms = max_over_ranks(ctx, statistics.median(chunks[len(chunks) // 2:]))  # the second half: after the clocks have come down
    tf = wl.work() / (ms * 1e-3) / 1e12  # per GPU
    peak = peaks["bf16_tflops_sustained"] / (6.0 if wl.bound == "tensor_f32" else 1.0)
    c = clk.summary()
    return {"value": round(tf * ctx.world, 2), "per_gpu": round(tf, 2), "unit": "TFLOP/s", "ms_per_step": round(ms, 4), "seconds": seconds,
            "roofline_frac": round(tf / peak, 4), "roofline_peak": round(peak, 1), "sm_mhz": c["sm_mhz"],
            "tflops_per_ghz": round(tf / (c["sm_mhz"] / 1e3), 1) if c["sm_mhz"] else None, "reasons": c["reasons"]}


NCU_TRAFFIC = {  # dram__bytes_read.sum + dram__bytes_write.sum per full-size launch (profiles/*.md)
    "softmax_f32": 4 * (268.5e6 + 215.7e6),       # captured on a quarter of the rows, scaled by rows
    "softmax_bf16": 4 * (134.2e6 + 79.0e6),
    "gemm_bf16_8192": 944.3e6 + 127.6e6,
    "gemm_f32_4096": 629.1e6 + 63.6e6 + 134.2e6 + 156.8e6,  # contraction + the two split kernels
    "attention_causal": 4 * (202.0e6 + 47.3e6),   # captured on 64 of 256 heads, scaled by heads
    "attention_noncausal": 4 * (201.4e6 + 49.2e6),
    "rms_norm_f32": 4 * (268.4e6 + 214.9e6),
    "reduce_sum_f32": 4 * (268.5e6 + 3.2e6),
    "silu_mul_f32": 4 * (536.9e6 + 229.3e6),
    "attention_decode_bf16": 4 * (537.0e6 + 4.6e6),
    "attention_f32_causal": 2 * (100.9e6 + 16.8e6),  # captured on 16 of 32 heads, scaled by heads
}


def measure(ctx, name, args, peaks, steps, warmup, headline=False, shared=None, keep=False):
    """Everything bench.py reports about one configuration.  Returns (record, workload or None)."""
    torch = _torch()
    wl = make_workload(ctx, name, args.units if headline else 0, shared=shared)
    reduced = bool(headline and args.units)
    scale = 1e9 if wl.bound == "hbm" else 1e12
    unit = "GB/s" if wl.bound == "hbm" else "TFLOP/s"
    torch.cuda.synchronize()
    time.sleep(0.3)  # let the power/clock state settle after the previous workload and the input set-up
    with ClockSampler(ctx.local) as clk:
        total_ms, per = time_steps(ctx, wl.step, steps, warmup)
    ms = total_ms / steps
    rec = {"value": round(ctx.world * wl.work() / (ms * 1e-3) / scale, 2), "unit": unit, "ms_per_step": round(ms, 4),
           "ms_per_step_min": round(min(per), 4), "ms_per_step_max": round(max(per), 4), "dtype": wl.dtype, "steps": steps}
    roof = roofline_for(wl, ms / wl.launches_per_step, peaks)
    roof["traffic"] = NCU_TRAFFIC.get(name)
    rec["roofline"] = roof
    rec["clocks"] = clk.summary()
    # strong scaling: this rank's shard of the SAME resident configuration (rows, problems, N columns, KV groups), timed
    # against the whole configuration in alternating blocks, so that both are timed at the same clocks and temperature
    # (one after the other, whichever ran second found the GPU hotter, or cooler after an oracle check, by 10 %)
    if name == "gemm_f32_512" and ctx.world > 1:
        rec["strong"] = {"note": "replicas only: 8 output tiles are too few to split; every GPU runs the same 512^3 problem"}
    elif ctx.world > 1 and not reduced and not isinstance(wl, (RowOpWL, DecodeWL)):
        sh = ctx.pkg.launcher.shard_range(wl.strong_units(), ctx.world, ctx.rank)
        if name.startswith("gemm_") and wl.single:
            sh = ctx.pkg.launcher.gemm_job(wl.code, wl.m, wl.n, wl.k, 0, 0, 0).plan(ctx.world, ctx.rank)
        fn = (lambda: wl.step_range(sh.first, sh.count)) if sh.count else (lambda: None)
        w_ms, s_ms = time_alternating(ctx, wl.step, fn, steps, 3)
        strong = {"value": round(wl.work() / (s_ms * 1e-3) / scale, 2), "unit": unit, "ms_per_step": round(s_ms, 4),
                  "one_gpu_ms_per_step": round(w_ms, 4), "speedup_vs_one_gpu": round(w_ms / s_ms, 3),
                  "split": wl.strong_unit or wl.unit_name, "this_rank": [int(sh.first), int(sh.count)], "of": int(wl.strong_units()),
                  "note": "blocks of 5 whole-configuration steps and of 5 shard steps alternate (same clocks and temperature "
                          "for both); every GPU carries the whole configuration in the former, its shard in the latter"}
        rec["strong"] = strong

    if wl.bound != "hbm" and args.sustained_seconds > 0 and not reduced:
        rec["sustained"] = sustained_run(ctx, wl, args.sustained_seconds, peaks, ctx.local)
        wl.step()
        torch.cuda.synchronize()

    # sampled check of this rank's result against the CPU oracle (untimed); the outcomes of all ranks are combined
    if hasattr(wl, "verify") and not args.no_verify and not reduced:
        v = wl.verify(ctx.oracle)
        v["ok"] = all_ranks_ok(ctx, v["ok"])
        v["ranks"] = ctx.world
        rec["verify"] = v
        assert v["ok"], f"{name}: verification against the CPU oracle failed: {v}"

    if "strong" in rec and "value" in rec["strong"] and hasattr(wl, "verify_strong") and not args.no_verify:
        strong = rec["strong"]
        sh_first, sh_count = strong["this_rank"]
        vs = wl.verify_strong(ctx.oracle, sh_first, sh_count) if sh_count else None
        if vs is not None:
            vs["ok"] = all_ranks_ok(ctx, vs["ok"])
            strong["verify"] = vs
            assert vs["ok"], f"{name}: the column block of rank {ctx.rank} does not match the oracle: {vs}"
        else:
            all_ranks_ok(ctx, True)

    # end to end through the host-buffer C-ABI call (pinned host memory, copies inside the timed region)
    if hasattr(wl, "e2e_prepare") and not args.no_e2e and not reduced:
        bi, bo, api = wl.e2e_prepare()
        wl.e2e_step()  # warm-up: allocates the staging workspace
        if ctx.world > 1:
            ctx.dist.barrier()
        n_e2e = 3 if wl.work() / scale > 3 else max(3, min(steps, 5))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            wl.e2e_step()
        dt = max_over_ranks(ctx, (time.perf_counter() - t0) / n_e2e)
        same = all_ranks_ok(ctx, wl.e2e_check())
        assert same, f"{name}: the host-buffer call and the device-buffer call disagree"
        rec["e2e"] = {"value": round(ctx.world * wl.work() / dt / scale, 2), "unit": unit, "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo,
                      "ms_per_step": round(dt * 1e3, 3), "steps": n_e2e, "api": api, "matches_device_path": same}
        if headline:
            rec["e2e"]["gbs_per_direction"] = round(ctx.world * bi / dt / 1e9, 1)
            rec["e2e"]["copy_probe"] = copy_probe(ctx)

    if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu_baseline and hasattr(wl, "cpu_run") and not reduced:
        v, sample = wl.cpu_run(ctx.oracle, args.cpu_seconds if headline else min(args.cpu_seconds, 5.0))
        rec["cpu_baseline"] = {"value": round(v, 4), "unit": unit, "cores": ctx.oracle.num_threads(), "kind": "port", "sample": sample}
    if name == "gemm_f32_512" and not reduced:
        # a latency-bound configuration: what one call costs the host, and the GPU, apart from the per-step event above
        n = 200
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            wl.step()
        host_us = (time.perf_counter() - t0) / n * 1e6  # the queue holds 200 small launches: nothing blocks
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            wl.step()
        e1.record()
        torch.cuda.synchronize()
        rec["latency"] = {"host_us_per_call": round(host_us, 2), "device_us_per_call_back_to_back": round(e0.elapsed_time(e1) / n * 1e3, 2),
                          "note": "host: Python + ctypes + launch, no synchronisation; device: 200 launches between two events"}
    if hasattr(wl, "context") and ctx.world == 1 and not reduced and not args.no_context:
        c = wl.context()
        if c:
            rec["context"] = c
    rec["config"] = config_for(name, args.units if headline else 0)
    rec["launches"] = steps * wl.launches_per_step
    if keep:
        return rec, wl
    wl.free()
    del wl
    torch.cuda.empty_cache()
    return rec, None


def run_ours(args):
    torch = _torch()
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    threads = host_threads(world)  # before the OpenMP users (input generator, oracle) are loaded
    ctx = Ctx()
    ctx.pkg = entry.load_package()
    ctx.hal, ctx.lib = ctx.pkg.hal, ctx.pkg.capi.lib()
    ctx.oracle = entry.load_oracle()  # the checker and the CPU-baseline leg; never part of a timed GPU step
    ctx.oracle.set_num_threads(threads)
    ctx.dev = ctx.hal.CudaSm100Device(local)
    ctx.tdev = torch.device(f"cuda:{local}")
    ctx.stream = torch.cuda.current_stream().cuda_stream
    ctx.world, ctx.rank, ctx.local, ctx.dist = world, rank, local, dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=ctx.tdev)
    peaks = measured_peaks()

    head, _ = measure(ctx, args.workload, args, peaks, args.steps, args.warmup, headline=True)
    extras, failed = {}, []
    if not args.no_extras:
        steps2 = max(3, min(args.steps, 10))
        names = [n for n in ORDER if n != args.workload]
        if args.only:
            names = [n for n in names if n in args.only.split(",")]
        shared_wl = None

        def guarded(name, **kw):
            """One configuration's failure (a check that does not hold, an out-of-memory box) is recorded under its
            name and in "failed"; the others are still measured and the line is still printed."""
            try:
                return measure(ctx, name, args, peaks, steps2, 3, **kw)
            except Exception as exc:  # noqa: BLE001
                if world > 1:
                    raise  # the other ranks would wait in a collective: fail the whole run instead
                torch.cuda.synchronize()
                torch.cuda.empty_cache()
                failed.append(name)
                return {"error": f"{type(exc).__name__}: {exc}"[:600]}, None

        for name in names:
            if name == "attention_noncausal" and "attention_causal" in names:
                # the causal configuration reads the same Q, K, V: keep them resident instead of generating them twice
                extras[name], shared_wl = guarded(name, keep=True)
                continue
            if name == "attention_causal" and shared_wl is not None:
                extras[name], _ = guarded(name, shared=shared_wl.shared())
                shared_wl.free()
                shared_wl = None
                torch.cuda.empty_cache()
                continue
            extras[name], _ = guarded(name)

    if rank == 0:
        def brief(r):
            if r is None:
                return None
            if "error" in r:
                return {"error": r["error"][:120]}
            b = {"value": r["value"], "unit": r["unit"], "ms": r["ms_per_step"], "frac": r["roofline"]["frac"]}
            if "sustained" in r:
                b["sust"], b["sust_frac"], b["per_ghz"] = r["sustained"]["value"], r["sustained"]["roofline_frac"], r["sustained"]["tflops_per_ghz"]
            if "verify" in r:
                b["verify"] = "ok" if r["verify"]["ok"] else "FAILED"
            if "cpu_baseline" in r:
                b["cpu"], b["cores"] = r["cpu_baseline"]["value"], r["cpu_baseline"]["cores"]
            if "e2e" in r:
                b["e2e"] = r["e2e"]["value"]
            if "strong" in r and "speedup_vs_one_gpu" in r["strong"]:
                b["strong_x"] = r["strong"]["speedup_vs_one_gpu"]
            if "context" in r and r["context"].get("torch_sdpa_tflops"):
                b["sdpa"] = r["context"]["torch_sdpa_tflops"]
            if "latency" in r:
                b["host_us"], b["dev_us"] = r["latency"]["host_us_per_call"], r["latency"]["device_us_per_call_back_to_back"]
            return b

        allrec = {args.workload: head, **extras}
        line = {
            "metric": METRIC if args.workload.startswith("softmax") else f"{args.workload} {head['unit']}",
            "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": head["dtype"], "data": "synthetic", "config": head["config"],
            "roofline": head["roofline"], "cpu_baseline": head.get("cpu_baseline"), "e2e": head.get("e2e"),
            "gpu_launches": head["launches"], "clocks": head["clocks"], "verify": head.get("verify"), "strong": head.get("strong"),
            "host_threads_per_rank": threads, "failed": failed,
            "workloads": extras,
            "summary": {n: brief(allrec.get(n)) for n in SUMMARY if n in allrec},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- reference arm
def reference_sample(name, rng):
    """(inputs, run(oracle), work per run, unit, description): a bounded sample of the configuration for the CPU."""
    cfg = catalogue_configs()[name]
    if name.startswith("softmax"):
        rows, cols = 2048, cfg["cols"]
        x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
        x[rng.random((rows, cols)) < 0.01] = 20.0
        if name.endswith("f32"):
            return (lambda o: o.softmax_f32(x)), rows * cols * 8, "GB/s", f"{rows} of {cfg['rows']} rows x {cols} cols per step (fits the CPU's caches: favours the CPU)"
        cache = {}

        def run16(o):
            if not cache:
                cache["x"] = o.f32_to_bf16(x)
            return o.softmax_bf16(cache["x"])
        return run16, rows * cols * 4, "GB/s", f"{rows} of {cfg['rows']} rows x {cols} cols per step (fits the CPU's caches: favours the CPU)"
    if name.startswith("gemm"):
        m, n, k = cfg["m"], cfg["n"], cfg["k"]
        f32 = "_f32_" in name
        rows = m if m <= 512 else 32
        if f32:
            a = (rng.random((rows, k)) * 2 - 1).astype(np.float32)
            b = (rng.random((k, n)) * 2 - 1).astype(np.float32)
            run = lambda o: o.gemm_f32(a, b)
        else:
            a32 = (rng.standard_normal((rows, k)) * k ** -0.25).astype(np.float32)
            b32 = (rng.standard_normal((k, n)) * k ** -0.25).astype(np.float32)
            cache = {}

            def run(o):
                if not cache:
                    cache["a"], cache["b"] = o.f32_to_bf16(a32), o.f32_to_bf16(b32)
                return o.gemm_bf16(cache["a"], cache["b"])
        what = "the whole problem" if rows == m else f"{rows} of {m} rows of C of one of {cfg['problems']} problem(s) against the full B per step (cost is linear in rows)"
        return run, 2.0 * rows * n * k, "TFLOP/s", what
    if name.startswith("attention") and name != "attention_decode_bf16":
        s, causal = cfg["seq"], cfg["causal"]
        q, k, v = (rng.standard_normal((1, 1, s, HEAD_DIM)).astype(np.float32) for _ in range(3))
        if "_f32_" in name:
            run = lambda o: o.attention_f32(q, k, v, causal)
        else:
            cache = {}

            def run(o):
                if not cache:
                    cache["t"] = tuple(o.f32_to_bf16(t) for t in (q, k, v))
                return o.attention_bf16(*cache["t"], causal)
        heads = cfg["batch"] * cfg["heads_q"]
        return run, 4.0 * s * s * HEAD_DIM * (0.5 if causal else 1.0), "TFLOP/s", f"1 of {heads} query heads at full sequence length per step (cost is linear in heads)"
    return None


def run_reference(args):
    """The reference's CPU path (its linalg semantics restated in oracle/) on all host threads.  Rank 0 alone runs it;
    it loads nothing but the oracle."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads(1)
    oracle = entry.load_oracle()
    oracle.set_num_threads(threads)
    rng = np.random.default_rng(2024)

    def time_one(name, steps, warmup):
        sample = reference_sample(name, rng)
        if sample is None:
            return None
        run, work, unit, what = sample
        for _ in range(warmup):
            run(oracle)
        t0 = time.perf_counter()
        for _ in range(steps):
            run(oracle)
        dt = (time.perf_counter() - t0) / steps
        return {"value": round(work / dt / (1e9 if unit == "GB/s" else 1e12), 4), "unit": unit, "ms_per_step": round(dt * 1e3, 3), "sample": what}

    head = time_one(args.workload, args.steps, args.warmup)
    if head is None:
        print(json.dumps({"impl": "reference", "unavailable": f"{args.workload} is a next-tier operator without a CPU leg in this arm"}))
        return
    extras, failed = {}, []
    if not args.no_extras:
        for name in ORDER:
            if name != args.workload:
                r = time_one(name, 2, 1)
                if r:
                    extras[name] = r
    cores = oracle.num_threads()
    line = {"impl": "reference", "metric": METRIC if args.workload.startswith("softmax") else f"{args.workload} {head['unit']}",
            "value": head["value"], "unit": head["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if "f32" in args.workload else "bf16",
            "data": "synthetic", "config": config_for(args.workload),
            "cpu_baseline": {"value": head["value"], "unit": head["unit"], "cores": cores, "kind": "port", "sample": head["sample"]},
            "e2e": {"value": head["value"], "unit": head["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "workloads": extras,
            "summary": {n: {"value": extras[n]["value"], "unit": extras[n]["unit"], "cores": cores} for n in SUMMARY if n in extras}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)  # 0.36 ms each: long enough for the clock sampler to see the load
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="softmax_f32", choices=sorted(catalogue_configs()))
    ap.add_argument("--scaling", default="weak", choices=["weak"],
                    help="the reported value is weak-scaled; the strong-scaling figure of every sharded configuration is reported beside it")
    ap.add_argument("--no-extras", action="store_true", help="measure only the headline workload")
    ap.add_argument("--only", default="", help="comma-separated subset of the other workloads to measure")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-context", action="store_true", help="skip the vendor-kernel yardstick of the attention workloads")
    ap.add_argument("--no-verify", action="store_true", help="skip the sampled check against the CPU oracle")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--sustained-seconds", type=float, default=1.5,
                    help="per tensor-bound workload: also a back-to-back loop of this length under the power cap (0: skip)")
    ap.add_argument("--units", type=int, default=0,
                    help="override the number of units (rows, problems, KV groups) per GPU of the headline workload: a reduced "
                         "case for profiler captures, never a benchmark number")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
