#!/usr/bin/env python
"""Benchmark of the tile-rs hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input that is
already resident in HBM.  The headline workload is the row softmax
configuration (65536 x 4096 f32, 3*N(0,1) with 1 % of the entries at +20); the
other configurations (bf16 softmax, bf16 GEMMs, f32 GEMM, attention forward)
are measured after it and reported under "workloads" in the same line.

Under torchrun (N > 1) every rank owns a shard of the units (rows, batches,
heads); there is no collective on the data path.  Times are CUDA-event times on
the launching stream, maximum over ranks.

--impl reference times the CPU restatement of the reference's linalg semantics
(the oracle) on the host cores for the same workload.
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
FP32_PIPE_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12  # FMA lanes x 2 flop x max clock


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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


# --------------------------------------------------------------------------- workloads
class Workload:
    """One configuration.  `units` are what is sharded over ranks; `work_per_unit` is the
    algorithmic bytes (HBM-bound) or flop (tensor-bound) of one unit."""
    name = ""
    bound = "hbm"          # or "tensor" / "fp32"
    dtype = "f32"
    unit_name = "rows"
    launches_per_step = 1

    def __init__(self, ctx, units: int):
        self.ctx, self.units = ctx, units

    def work(self) -> float:
        return self.units * self.work_per_unit

    def describe(self) -> dict:
        return {}


def _torch():
    import torch
    return torch


class SoftmaxWL(Workload):
    unit_name = "rows"

    def __init__(self, ctx, units, dtype="f32", first_unit=0, host_inputs=True):
        super().__init__(ctx, units)
        torch, capi = _torch(), ctx.pkg.capi
        self.dtype, self.cols = dtype, SOFTMAX_COLS
        self.name = f"softmax_{dtype}"
        self.es = 4 if dtype == "f32" else 2
        self.code = capi.F32 if dtype == "f32" else capi.BF16
        self.work_per_unit = self.cols * self.es * 2  # one read + one write per element
        n = units * self.cols
        self.x_host = None
        if host_inputs:
            lib = capi.lib()
            ptr = C.c_void_p()
            ctx.hal.check(lib.tsm100_host_alloc(n * 4, C.byref(ptr)))
            x = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(n,))
            lib.tsm100_fill_normal_f32(ptr, n, 201, first_unit * self.cols, 3.0)
            lib.tsm100_plant_outliers_f32(ptr, n, 202, first_unit * self.cols, 100, 20.0)
            self.x_host, self._x_ptr = x, ptr
            xd = torch.empty(n, dtype=torch.float32, device=ctx.tdev)
            ctx.hal.check(lib.tsm100_memcpy_h2d(ctx.dev._h, xd.data_ptr(), ptr, n * 4, None))
            torch.cuda.synchronize()
        else:
            g = torch.Generator(device=ctx.tdev).manual_seed(201 + first_unit)
            xd = torch.randn(n, device=ctx.tdev, generator=g) * 3
            xd[torch.rand(n, device=ctx.tdev, generator=g) < 0.01] = 20.0
        self.x = xd if dtype == "f32" else xd.to(torch.bfloat16)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.ctx.dev.softmax(self.code, self.units, self.cols, self.x.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)

    def describe(self):
        return {"rows_per_gpu": self.units, "cols": self.cols, "law": "3*N(0,1), 1% of entries = +20"}

    # end to end: pinned host buffers in, pinned host buffers out, through tsm100_softmax_host
    def e2e_prepare(self):
        lib = self.ctx.pkg.capi.lib()
        n = self.units * self.cols
        self._y_ptr = C.c_void_p()
        self.ctx.hal.check(lib.tsm100_host_alloc(n * 4, C.byref(self._y_ptr)))
        return n * 4, n * 4

    def e2e_step(self):
        self.ctx.dev.softmax_host(self.code, self.units, self.cols, self._x_ptr.value, self._y_ptr.value)

    def e2e_check(self):
        y = np.ctypeslib.as_array(C.cast(self._y_ptr, C.POINTER(C.c_float)), shape=(self.units, self.cols))
        s = y[:: max(1, self.units // 64)].sum(axis=1)
        assert np.abs(s - 1).max() < 1e-4, "end-to-end softmax rows do not sum to one"

    def cpu_run(self, oracle, seconds: float):
        rows = min(self.units, 4096)
        x = self.x_host[: rows * self.cols].reshape(rows, self.cols)
        t_end, done, t0 = time.perf_counter() + seconds, 0, time.perf_counter()
        while True:
            oracle.softmax_f32(x)
            done += rows
            if time.perf_counter() >= t_end:
                break
        dt = time.perf_counter() - t0
        return done * self.work_per_unit / dt / 1e9, f"{rows} rows x {self.cols} cols f32, {done // rows} passes in {dt:.1f} s"


class RowOpWL(Workload):
    """rms_norm / row sum / silu * mul on the softmax configuration's shape (rows x 4096)."""
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
        if op == "reduce_sum":
            self.y = torch.empty(units, device=ctx.tdev, dtype=tdt)
        else:
            self.y = torch.empty_like(self.x)
        self.up = torch.randn(units, self.cols, device=ctx.tdev, generator=g).to(tdt) if op == "silu_mul" else None

    def step(self):
        d, capi = self.ctx.dev, self.ctx.pkg.capi
        if self.op == "rms_norm":
            d.rms_norm(self.code, self.units, self.cols, 1e-5, self.x.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)
        elif self.op == "reduce_sum":
            d.reduce(self.code, capi.REDUCE_SUM, self.units, self.cols, self.x.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)
        else:
            d.silu_mul(self.code, self.units, self.cols, self.x.data_ptr(), self.up.data_ptr(), self.y.data_ptr(), stream=self.ctx.stream)

    def describe(self):
        return {"cols": self.cols, "rows_per_gpu": self.units}


class GemmWL(Workload):
    bound, unit_name = "tensor", "problems"

    def __init__(self, ctx, units, m, n, k, dtype="bf16", name=None):
        super().__init__(ctx, units)
        torch, capi = _torch(), ctx.pkg.capi
        self.m, self.n, self.k, self.dtype = m, n, k, dtype
        self.name = name or f"gemm_{dtype}_{m}x{n}x{k}"
        self.work_per_unit = 2.0 * m * n * k
        g = torch.Generator(device=ctx.tdev).manual_seed(301)
        if dtype == "f32":
            self.bound, self.code = "fp32", capi.F32
            self.a = torch.rand(units, m, k, device=ctx.tdev, generator=g) * 2 - 1
            self.b = torch.rand(units, k, n, device=ctx.tdev, generator=g) * 2 - 1
            self.c = torch.empty(units, m, n, device=ctx.tdev)
        else:
            self.code = capi.BF16
            sigma = k ** -0.25  # variance 1/sqrt(K): outputs are O(1)
            self.a = (torch.randn(units, m, k, device=ctx.tdev, generator=g) * sigma).to(torch.bfloat16)
            self.b = (torch.randn(units, k, n, device=ctx.tdev, generator=g) * sigma).to(torch.bfloat16)
            self.c = torch.empty(units, m, n, device=ctx.tdev, dtype=torch.bfloat16)

    def step(self):
        self.ctx.dev.gemm(self.code, self.m, self.n, self.k, self.a.data_ptr(), self.b.data_ptr(), self.c.data_ptr(),
                          batch=self.units, stream=self.ctx.stream)

    def describe(self):
        return {"m": self.m, "n": self.n, "k": self.k, "problems_per_gpu": self.units}


class AttentionWL(Workload):
    bound, unit_name, dtype = "tensor", "kv_groups", "bf16"

    def __init__(self, ctx, units, group, seq, causal, name, dtype="bf16"):
        super().__init__(ctx, units)
        torch = _torch()
        self.group, self.seq, self.causal, self.name, self.dtype = group, seq, causal, name, dtype
        if dtype == "f32":  # three TF32 products per product on the warp-level MMA: compared with the FP32 FMA rate
            self.bound = "fp32"
        self.work_per_unit = 4.0 * group * seq * seq * 128 * (0.5 if causal else 1.0)
        g = torch.Generator(device=ctx.tdev).manual_seed(401)
        mk = lambda h: torch.randn(units, h, seq, 128, device=ctx.tdev, generator=g).to(torch.float32 if dtype == "f32" else torch.bfloat16)
        self.q, self.k, self.v = mk(group), mk(1), mk(1)
        self.o = torch.empty_like(self.q)

    def step(self):
        capi = self.ctx.pkg.capi
        self.ctx.dev.attention(capi.F32 if self.dtype == "f32" else capi.BF16, self.units, self.group, 1, self.seq, 128, self.q.data_ptr(),
                               self.k.data_ptr(), self.v.data_ptr(), self.o.data_ptr(), causal=self.causal,
                               stream=self.ctx.stream)

    def describe(self):
        return {"q_heads_per_kv_head": self.group, "seq": self.seq, "head_dim": 128, "causal": self.causal,
                "kv_groups_per_gpu": self.units}


class DecodeWL(Workload):
    """One decode step: `units` (batch, KV head) caches of 16384 x 128 bf16, 8 query heads each."""
    unit_name = "kv_caches"
    bound = "hbm"
    dtype = "bf16"

    def __init__(self, ctx, units, seq=16384, group=8, name="attention_decode_bf16"):
        super().__init__(ctx, units)
        torch = _torch()
        self.seq, self.group, self.name = seq, group, name
        g = torch.Generator(device=ctx.tdev).manual_seed(801)
        self.q = torch.randn(units, group, 128, device=ctx.tdev, generator=g).to(torch.bfloat16)
        self.k = torch.randn(units, 1, seq, 128, device=ctx.tdev, generator=g).to(torch.bfloat16)
        self.v = torch.randn(units, 1, seq, 128, device=ctx.tdev, generator=g).to(torch.bfloat16)
        self.o = torch.empty_like(self.q)
        self.work_per_unit = 2.0 * seq * 128 * 2 + 2.0 * group * 128 * 2  # K and V once, q in, o out

    def step(self):
        self.ctx.dev.attention_decode(self.ctx.pkg.capi.BF16, self.units, self.group, 1, self.seq, self.seq, 128,
                                      self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.o.data_ptr(),
                                      stream=self.ctx.stream)

    def describe(self):
        return {"q_heads_per_kv_head": self.group, "seq_len": self.seq, "head_dim": 128, "kv_caches_per_gpu": self.units}


# name -> (units at one GPU, factory(ctx, units, first_unit))
def catalogue():
    return {
        "softmax_f32": (SOFTMAX_ROWS, lambda c, u, f: SoftmaxWL(c, u, "f32", f)),
        "softmax_bf16": (SOFTMAX_ROWS, lambda c, u, f: SoftmaxWL(c, u, "bf16", f, host_inputs=False)),
        "gemm_bf16_8192": (1, lambda c, u, f: GemmWL(c, u, 8192, 8192, 8192, name="gemm_bf16_8192")),
        "gemm_bf16_batched_4096": (64, lambda c, u, f: GemmWL(c, u, 4096, 4096, 4096, name="gemm_bf16_batched_4096")),
        "gemm_f32_512": (1, lambda c, u, f: GemmWL(c, u, 512, 512, 512, "f32", name="gemm_f32_512")),
        "attention_noncausal": (256, lambda c, u, f: AttentionWL(c, u, 1, 4096, False, "attention_noncausal")),
        "attention_causal": (256, lambda c, u, f: AttentionWL(c, u, 1, 4096, True, "attention_causal")),
        "attention_gqa_causal": (16, lambda c, u, f: AttentionWL(c, u, 8, 16384, True, "attention_gqa_causal")),
        "attention_f32_causal": (32, lambda c, u, f: AttentionWL(c, u, 1, 4096, True, "attention_f32_causal", "f32")),
        "rms_norm_f32": (SOFTMAX_ROWS, lambda c, u, f: RowOpWL(c, u, "rms_norm")),
        "reduce_sum_f32": (SOFTMAX_ROWS, lambda c, u, f: RowOpWL(c, u, "reduce_sum")),
        "silu_mul_f32": (SOFTMAX_ROWS, lambda c, u, f: RowOpWL(c, u, "silu_mul")),
        "silu_mul_bf16": (SOFTMAX_ROWS, lambda c, u, f: RowOpWL(c, u, "silu_mul", "bf16")),
        "attention_decode_bf16": (256, lambda c, u, f: DecodeWL(c, u)),
    }


class Ctx:
    pass


def time_steps(ctx, wl, steps, warmup):
    """Returns (total ms over `steps`, list of per-step ms), device-timed on the launching stream."""
    torch = _torch()
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        wl.step()
        evs[i + 1].record()
    torch.cuda.synchronize()
    if ctx.world > 1:
        ctx.dist.barrier()
    total = evs[0].elapsed_time(evs[-1])
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    if ctx.world > 1:
        t = torch.tensor([total], device=ctx.tdev, dtype=torch.float64)
        ctx.dist.all_reduce(t, op=ctx.dist.ReduceOp.MAX)
        total = float(t.item())
    assert ctx.dev.status() == 0, "a kernel reported a timed-out device-side wait"
    return total, per


def roofline_for(wl, ms_per_launch, peaks):
    if wl.bound == "hbm":
        achieved, peak, unit = wl.work() / (ms_per_launch * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    elif wl.bound == "tensor":
        achieved, peak, unit = wl.work() / (ms_per_launch * 1e-3) / 1e12, peaks["bf16_tflops"], "TFLOP/s"
    else:
        achieved, peak, unit = wl.work() / (ms_per_launch * 1e-3) / 1e12, FP32_PIPE_PEAK_TFLOPS, "TFLOP/s"
    return {"bound": "hbm" if wl.bound == "hbm" else "tensor" if wl.bound == "tensor" else "fp32", "achieved": round(achieved, 2),
            "peak": round(peak, 2), "unit": unit, "frac": round(achieved / peak, 4),
            "peak_source": peaks["source"] if wl.bound != "fp32" else "nominal FP32 FMA rate at max clock"}


def sustained_run(ctx, wl, seconds, global_units, peaks, gpu_index):
    """The tensor-bound kernels draw the board's full power: the short timed run above sees burst clocks, a
    loop of a second or more runs under the power cap.  Launches back to back for `seconds`, timed on the
    device, with the clock sampler running; the fraction is of the measured sustained GEMM peak."""
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
    ms = statistics.median(chunks[len(chunks) // 2:])  # the second half: after the clocks have come down
    tf = global_units * wl.work_per_unit / (ms * 1e-3) / 1e12
    return {"value": round(tf, 2), "unit": "TFLOP/s", "ms_per_step": round(ms, 4), "seconds": seconds,
            "roofline_frac": round(tf / peaks["bf16_tflops_sustained"], 4), "roofline_peak": peaks["bf16_tflops_sustained"],
            "clocks": clk.summary()}


NCU_TRAFFIC = {  # dram__bytes_read.sum + dram__bytes_write.sum per full-size launch (profiles/*.md)
    "softmax_f32": 4 * (268.5e6 + 215.7e6),       # captured on a quarter of the rows, scaled by rows
    "softmax_bf16": 4 * (134.2e6 + 79.0e6),
    "gemm_bf16_8192": 1064.7e6 + 127.0e6,
    "attention_causal": 4 * (201.4e6 + 48.2e6),   # captured on 64 of 256 heads, scaled by heads
    "attention_noncausal": 4 * (201.4e6 + 48.0e6),
    "rms_norm_f32": 4 * (268.4e6 + 214.9e6),
    "reduce_sum_f32": 4 * (268.5e6 + 3.2e6),
    "silu_mul_f32": 4 * (536.9e6 + 229.3e6),
    "attention_decode_bf16": 4 * (537.0e6 + 4.6e6),
    "attention_f32_causal": 2 * (100.9e6 + 16.8e6),  # captured on 16 of 32 heads, scaled by heads
}


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
    if world > 1:  # torchrun pins OMP_NUM_THREADS=1; the host input generator may use this rank's share of the cores
        os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or world) // world))
    ctx = Ctx()
    ctx.pkg = entry.load_package()
    ctx.hal = ctx.pkg.hal
    ctx.dev = ctx.hal.CudaSm100Device(local)
    ctx.tdev = torch.device(f"cuda:{local}")
    ctx.stream = torch.cuda.current_stream().cuda_stream
    ctx.world, ctx.rank, ctx.dist = world, rank, dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=ctx.tdev)
    peaks = measured_peaks()
    cat = catalogue()
    base_units, factory = cat[args.workload]
    if args.units:
        base_units = args.units  # reduced case, for profiler captures only
    # weak scaling: every GPU carries the one-GPU configuration; strong: the configuration is split
    if args.scaling == "weak":
        units, first = base_units, rank * base_units
    else:
        sh = ctx.pkg.shard.shard_range(base_units, world, rank)
        units, first = sh.count, sh.first
    wl = factory(ctx, units, first)

    with ClockSampler(local) as clk:
        total_ms, per = time_steps(ctx, wl, args.steps, args.warmup)
    ms_per_step = total_ms / args.steps
    global_units = base_units * world if args.scaling == "weak" else base_units
    global_work = global_units * wl.work_per_unit
    scale = 1e9 if wl.bound == "hbm" else 1e12
    value = global_work / (ms_per_step * 1e-3) / scale
    unit = "GB/s" if wl.bound == "hbm" else "TFLOP/s"
    roof = roofline_for(wl, statistics.mean(per) / wl.launches_per_step, peaks)
    roof["traffic"] = NCU_TRAFFIC.get(wl.name)

    # verification (untimed): a few rows of every rank's shard, gathered over NCCL when there are several
    # ranks, against the CPU oracle on rank 0 - the one use of a collective, and not on the data path
    verify = None
    if isinstance(wl, SoftmaxWL) and not args.no_verify:
        idx = torch.tensor(sorted({0, units // 2, units - 1}), device=ctx.tdev)
        xs, ys = wl.x.view(units, -1)[idx].contiguous(), wl.y.view(units, -1)[idx].contiguous()
        if world > 1:
            gx = [torch.empty_like(xs) for _ in range(world)]
            gy = [torch.empty_like(ys) for _ in range(world)]
            dist.all_gather(gx, xs)
            dist.all_gather(gy, ys)
            xs, ys = torch.cat(gx), torch.cat(gy)
        if rank == 0:
            oracle = entry.load_oracle()
            if wl.dtype == "f32":
                ref = oracle.softmax_f32(xs.cpu().numpy(), f64_acc=True)
                got = ys.cpu().numpy()
                tol = 1e-5
            else:
                ref, _ = oracle.softmax_bf16(xs.view(torch.int16).cpu().numpy().view(np.uint16))
                got = oracle.bf16_to_f32(ys.view(torch.int16).cpu().numpy().view(np.uint16))
                tol = 2.0 ** -8
            err = float(np.abs(got - ref).max() / np.abs(ref).max())
            assert err <= tol, f"verification against the oracle failed: {err}"
            verify = {"rows": int(xs.shape[0]), "ranks": world, "max_err_rel_to_max": err, "tolerance": tol,
                      "against": "CPU oracle (float64-accumulating)" if wl.dtype == "f32" else "CPU oracle"}

    # end to end through the host-buffer C-ABI call (pinned host memory, copies inside the timed region)
    e2e = None
    if hasattr(wl, "e2e_prepare") and not args.no_e2e:
        bi, bo = wl.e2e_prepare()
        wl.e2e_step()  # warm-up: allocates the staging workspace
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        n_e2e = max(2, min(args.steps, 5))
        for _ in range(n_e2e):
            wl.e2e_step()
        dt = (time.perf_counter() - t0) / n_e2e
        if world > 1:
            t = torch.tensor([dt], device=ctx.tdev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        wl.e2e_check()
        e2e = {"value": round(global_work / dt / scale, 2), "unit": unit, "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo,
               "ms_per_step": round(dt * 1e3, 3), "api": "tsm100_softmax_host (pinned host buffers, chunked copy/compute overlap)"}

    # the other configurations, one after another, same timing rules
    extras = {}
    if not args.no_extras:
        del wl.x, wl.y
        torch.cuda.empty_cache()
        for name, (bu, fac) in cat.items():
            if name == args.workload:
                continue
            if args.scaling == "weak":
                u, f = bu, rank * bu
            else:
                sh = ctx.pkg.shard.shard_range(bu, world, rank)
                u, f = sh.count, sh.first
            if u == 0:
                continue
            w2 = fac(ctx, u, f)
            torch.cuda.synchronize()
            time.sleep(0.5)  # let the power/clock state settle after the previous workload and the input set-up
            steps2 = max(3, min(args.steps, 10))
            tot, per2 = time_steps(ctx, w2, steps2, 3)
            ms = tot / steps2
            gu = bu * world if args.scaling == "weak" else bu
            sc = 1e9 if w2.bound == "hbm" else 1e12
            r2 = roofline_for(w2, statistics.mean(per2), peaks)
            extras[name] = {"value": round(gu * w2.work_per_unit / (ms * 1e-3) / sc, 2), "unit": "GB/s" if w2.bound == "hbm" else "TFLOP/s",
                            "ms_per_step": round(ms, 4), "ms_per_step_min": round(min(per2), 4), "ms_per_step_max": round(max(per2), 4), "dtype": w2.dtype, "roofline_frac": r2["frac"], "roofline_peak": r2["peak"],
                            "config": w2.describe()}
            if w2.bound == "tensor" and args.sustained_seconds > 0:
                extras[name]["sustained"] = sustained_run(ctx, w2, args.sustained_seconds, gu, peaks, local)
            del w2
            torch.cuda.empty_cache()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and hasattr(wl, "cpu_run"):
        oracle = entry.load_oracle()
        v, sample = wl.cpu_run(oracle, args.cpu_seconds)
        cpu = {"value": round(v, 3), "unit": unit, "cores": oracle.num_threads(), "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": "row softmax HBM GB/s (GEMM / attention TFLOP/s under 'workloads')" if wl.bound == "hbm" else f"{wl.name} TFLOP/s",
            "value": round(value, 2), "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.name + (" (REDUCED: --units)" if args.units else ""), **wl.describe(), "global_units": global_units, "unit": wl.unit_name,
                       "l2": "inputs larger than L2 (no flush needed)" if wl.work() > 300e6 else "inputs fit in L2",
                       "sharding": f"{wl.unit_name} split over ranks, no collective on the data path"},
            "roofline": roof, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": args.steps * wl.launches_per_step, "clocks": clk.summary(), "verify": verify, "workloads": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU path (its linalg semantics restated in oracle/) on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pkg = entry.load_package()
    oracle = entry.load_oracle()
    capi = pkg.capi
    if args.workload != "softmax_f32":
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm implemented for softmax_f32, not {args.workload}"}))
        return
    rows, cols = 2048, SOFTMAX_COLS  # bounded sample of the 65536-row configuration per step
    x = np.empty((rows, cols), np.float32)
    capi.lib().tsm100_fill_normal_f32(x.ctypes.data, x.size, 201, 0, 3.0)
    capi.lib().tsm100_plant_outliers_f32(x.ctypes.data, x.size, 202, 0, 100, 20.0)
    for _ in range(args.warmup):
        oracle.softmax_f32(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.softmax_f32(x)
    dt = (time.perf_counter() - t0) / args.steps
    value = rows * cols * 8 / dt / 1e9
    sample = f"{rows} of {SOFTMAX_ROWS} rows x {cols} cols f32 per step"
    line = {"impl": "reference", "metric": "row softmax HBM GB/s (GEMM / attention TFLOP/s under 'workloads')",
            "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "softmax_f32", "rows_per_gpu": SOFTMAX_ROWS, "cols": cols, "law": "3*N(0,1), 1% of entries = +20"},
            "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)  # 0.36 ms each: long enough for the clock sampler to see the load
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="softmax_f32", choices=sorted(catalogue()))
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-extras", action="store_true", help="measure only the headline workload")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true", help="skip the sampled-rows check against the CPU oracle")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--sustained-seconds", type=float, default=1.5,
                    help="per tensor-bound workload: also a back-to-back loop of this length under the power cap (0: skip)")
    ap.add_argument("--units", type=int, default=0,
                    help="override the number of units (rows, problems, KV groups) per GPU: a reduced case for "
                         "profiler captures, never a benchmark number")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
